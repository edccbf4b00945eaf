#!/usr/bin/env python3
"""Test infrastructure: build the UNMODIFIED reference `quant` extension for sm_100a.

The reference (sparklesea/sparse-quant, quantization/nvidia) ships its W4A16 path as a
torch C++/CUDA extension named `quant` (kernel/pybind.cpp, kernel/gemm_quant.cu,
kernel/gemm_s4_f16/format.cu, kernel/gemm_s4_f16/gemm_s4_f16.cu; build flags from
quantization/nvidia/setup.py:64-70, which passes no -gencode at all).  This recipe compiles
those four sources *where they lie* (nothing is copied) with the reference's own flags plus
`-gencode arch=compute_100a,code=sm_100a`, and links the result into

    oracle/_ref/quant.cpython-*.so

That module is a GPU comparator for the parity tests (layout kernels byte-for-byte, the
identity-matrix dequant trick, GEMM outputs) and the generator of the golden vectors under
tests/golden/.  It is never imported by the product.

It also stages, unmodified and again only into the untracked oracle/_ref/, the three Python
files of the reference that sit directly on top of the `quant` extension
(test/nvidia/module/qlinear/qlinear.py, test/nvidia/utils/quant_dequant_nvidia.py,
test/nvidia/utils/quant_funcs.py) under oracle/_ref/refpy/ with their package layout, so that
tests/test_gpu_dropin_reference_python.py can run the reference's own WALinear on this
library's `quant` module.

Usage:  python oracle/build_ref.py [--reference /path/to/reference] [--jobs 4]
Exits 0 and does nothing if the reference tree is absent (the GPU box only uses the
prebuilt file) or the module is already built and newer than its sources.
"""
import argparse
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
SOURCES = [
    "kernel/pybind.cpp",
    "kernel/gemm_quant.cu",
    "kernel/gemm_s4_f16/format.cu",
    "kernel/gemm_s4_f16/gemm_s4_f16.cu",
]


PY_FILES = [
    "module/qlinear/qlinear.py",
    "utils/quant_dequant_nvidia.py",
    "utils/quant_funcs.py",
]


def stage_python(reference, verbose=True):
    """Copy the reference's WALinear and quantizer Python (unmodified) to oracle/_ref/refpy/."""
    import shutil
    src_root = os.path.join(reference, "test", "nvidia")
    if not os.path.isdir(src_root):
        return None
    dst_root = os.path.join(OUT, "refpy")
    for rel in PY_FILES:
        src, dst = os.path.join(src_root, rel), os.path.join(dst_root, rel)
        if not os.path.exists(src):
            if verbose:
                print(f"[build_ref] missing {src}")
            return None
        os.makedirs(os.path.dirname(dst), exist_ok=True)
        if not os.path.exists(dst) or os.path.getmtime(dst) < os.path.getmtime(src):
            shutil.copyfile(src, dst)
    return dst_root


def target_path():
    return os.path.join(OUT, "quant" + sysconfig.get_config_var("EXT_SUFFIX"))


def build(reference, jobs=4, verbose=True):
    src_root = os.path.join(reference, "quantization", "nvidia")
    if not os.path.isdir(src_root):
        if verbose:
            print(f"[build_ref] no reference tree at {src_root}; nothing to do")
        return None
    srcs = [os.path.join(src_root, s) for s in SOURCES]
    tgt = target_path()
    stage_python(reference, verbose)
    if os.path.exists(tgt) and all(os.path.getmtime(tgt) >= os.path.getmtime(s) for s in srcs):
        if verbose:
            print(f"[build_ref] up to date: {tgt}")
        return tgt

    import torch
    from torch.utils import cpp_extension as ce

    os.makedirs(OUT, exist_ok=True)
    incs = ce.include_paths("cuda") + [sysconfig.get_paths()["include"]]
    inc_flags = [f"-I{p}" for p in incs]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    common = [
        "-DTORCH_EXTENSION_NAME=quant", "-DTORCH_API_INCLUDE_EXTENSION_H",
        f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-DBUILD_WITH_CUDA",
    ]
    nvcc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")

    def compile_one(src):
        obj = os.path.join(OUT, os.path.basename(src) + ".o")
        if src.endswith(".cu"):
            cmd = [nvcc, "-c", src, "-o", obj, "-O3", "-std=c++17", "--generate-line-info",
                   "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__",
                   "--expt-relaxed-constexpr",
                   "-gencode", "arch=compute_100a,code=sm_100a",
                   "-Xcompiler", "-fPIC"] + common + inc_flags
        else:
            cmd = ["g++", "-c", src, "-o", obj, "-O3", "-std=c++17", "-fPIC", "-fopenmp"] + common + inc_flags
        if verbose:
            print("[build_ref]", " ".join(cmd[:6]), "...")
        subprocess.check_call(cmd)
        return obj

    with ThreadPoolExecutor(max_workers=jobs) as ex:
        objs = list(ex.map(compile_one, srcs))

    lib_dirs = ce.library_paths("cuda") if "device_type" in ce.library_paths.__code__.co_varnames else ce.library_paths(True)
    link = ["g++", "-shared", "-o", tgt] + objs
    for d in lib_dirs:
        link += [f"-L{d}", f"-Wl,-rpath,{d}"]
    link += ["-lc10", "-ltorch_cpu", "-ltorch", "-ltorch_python", "-lc10_cuda", "-ltorch_cuda", "-lcudart", "-lgomp"]
    subprocess.check_call(link)
    for o in objs:
        os.remove(o)
    if verbose:
        print(f"[build_ref] built {tgt}")
    return tgt


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("W4A16_REFERENCE", ""),
                    help="root of the reference tree (or set W4A16_REFERENCE)")
    ap.add_argument("--jobs", type=int, default=4)
    a = ap.parse_args()
    if not a.reference:
        print("[build_ref] no reference tree given (--reference or W4A16_REFERENCE); nothing to do")
        sys.exit(0)
    build(a.reference, a.jobs)
    sys.exit(0)
