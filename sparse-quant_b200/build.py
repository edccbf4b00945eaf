#!/usr/bin/env python3
"""Build libw4a16_b200.so (sm_100a only) in-tree with nvcc.

    python sparse-quant_b200/build.py [--force] [--verbose]

The shared library exposes the C ABI declared in include/w4a16_b200.h and is loaded by the
`quant` Python package with ctypes.  nvcc cross-compiles without a GPU.
"""
import argparse
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "quant", "libw4a16_b200.so")


def sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def up_to_date():
    if not os.path.exists(OUT):
        return False
    deps = sources() + glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(ROOT, "include", "*.h"))
    return all(os.path.getmtime(OUT) >= os.path.getmtime(d) for d in deps)


def build(force=False, verbose=False):
    if not force and up_to_date():
        return OUT
    nvcc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    cmd = [nvcc, "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
           "-Xcompiler", "-fPIC", "-shared", "--threads", "0",
           "-I", os.path.join(ROOT, "include"), "-I", CSRC, "-o", OUT] + sources()
    if os.environ.get("W4A16_DEBUG"):
        cmd.insert(1, "-DW4A16_SKINNY_DEBUG")    # phase time stamps / experiment switches in the decode kernel
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
        print(" ".join(cmd))
    subprocess.check_call(cmd)
    return OUT


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
    sys.exit(0)
