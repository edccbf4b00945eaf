"""The C-ABI library loads and exports every symbol include/w4a16_b200.h declares; argument
errors come back as status codes before anything touches a GPU; the Python `quant` shim raises
RuntimeError the way the reference's TORCH_CHECKs do.  No compute call is made here."""
import ctypes
import os
import re

import pytest
import torch

import quant

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "w4a16_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(w4a16_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = quant.load_library()
    names = declared_symbols()
    assert len(names) >= 12
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/w4a16_b200.h but not exported"
    assert set(names) == set(quant.C_ABI), "ctypes table and header disagree"
    assert lib.w4a16_version() >= 100
    assert lib.w4a16_status_str(0) == b"success"
    assert lib.w4a16_status_str(3) == b"unsupported group size"


def test_status_codes_without_a_gpu():
    lib = quant.load_library()
    buf = (ctypes.c_char * 4096)()
    p = ctypes.addressof(buf)
    p = (p + 15) & ~15
    # group size the format does not support -> the reference's "unsupported group size"
    assert lib.w4a16_gemm(p, p, p, None, p, 1, 64, 128, 100, None, 0, None) == 3
    # N not a multiple of 32, K not a multiple of g, negative tokens
    assert lib.w4a16_gemm(p, p, p, None, p, 1, 48, 128, 128, None, 0, None) == 2
    assert lib.w4a16_gemm(p, p, p, None, p, 1, 64, 192, 128, None, 0, None) == 2
    assert lib.w4a16_gemm(p, p, p, None, p, -1, 64, 128, 128, None, 0, None) == 2
    # NULL / misaligned pointers
    assert lib.w4a16_gemm(None, p, p, None, p, 1, 64, 128, 128, None, 0, None) == 1
    assert lib.w4a16_gemm(p + 2, p, p, None, p, 1, 64, 128, 128, None, 0, None) == 4
    # zero tokens is a successful no-op
    assert lib.w4a16_gemm(None, None, None, None, None, 0, 64, 128, 128, None, 0, None) == 0
    assert lib.w4a16_gemm_algo(p, p, p, None, p, 1, 64, 128, 128, None, 0, None, 9) == 6
    assert lib.w4a16_dequant(p, p, p, 64, 128, 96, None) == 3
    assert lib.w4a16_dequant(p, p, p, 40, 128, 128, None) == 2
    assert lib.w4a16_convert_awq_to_lmdeploy(p, p + 2048, 100, 64, None) == 2
    assert lib.w4a16_convert_awq_to_lmdeploy(p, p, 128, 64, None) == 2          # in place is rejected
    assert lib.w4a16_convert_ours_to_awq(None, p, 128, 64, None) == 1
    assert lib.w4a16_transpose_merge_zeros_scales(p, p, p, 128, 64, 0, None) == 3
    assert lib.w4a16_workspace_bytes(1, 4096, 4096, 128) == 0


def test_python_shim_rejects_like_the_reference():
    I = torch.zeros(1, 1, 128, dtype=torch.float16)
    W = torch.zeros(128, 8, dtype=torch.int32)
    ZS = torch.zeros(1, 128, dtype=torch.float16)
    with pytest.raises(RuntimeError, match="must be on CUDA"):
        quant.gemm_awq_ut(I, W, ZS, 1, 64, 128, 128)
    with pytest.raises(RuntimeError):
        quant.dequant(W, ZS, 64, 128, 128)
    with pytest.raises(RuntimeError):
        quant.transpose_merge_zeros_scales(ZS, ZS, ZS, 128, 64, 128)
