"""TEST INFRASTRUCTURE — the parity checker, not the product.

CPU oracle for the W4A16 path of sparklesea/sparse-quant's `quant` extension.  The
arithmetic lives in ``w4a16_oracle.c`` (plain C, bit-level fp16 emulation, every function
citing the reference file:line it restates); this module loads it with ctypes and exposes
numpy-level wrappers, plus a torch-CPU restatement of the reference's Python quantizer.

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline / reference legs of
``bench.py`` may import this package.  Nothing in the product does.

Parity pin: ``tests/test_oracle_golden.py`` checks these functions against vectors made by
the reference's own Python (imported on CPU) and by the reference's own CUDA extension
(rebuilt for sm_100a, run on a B200); see ``tests/golden/make_golden.py``.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libw4a16_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile the C restatement (gcc, seconds)."""
    src = os.path.join(_HERE, "w4a16_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "libw4a16_oracle.so"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(_LIB_PATH)
        vp, ci = ctypes.c_void_p, ctypes.c_int
        L.oracle_convert_ours_to_awq.argtypes = [vp, vp, ci, ci]
        L.oracle_convert_awq_to_lmdeploy.argtypes = [vp, vp, ci, ci]
        L.oracle_transpose_merge_zeros_scales.argtypes = [vp, vp, vp, ci, ci, ci]
        L.oracle_unpack.argtypes = [vp, vp, ci, ci]
        L.oracle_dequant.argtypes = [vp, vp, vp, ci, ci, ci]
        L.oracle_dequant_f32.argtypes = [vp, vp, vp, ci, ci, ci]
        L.oracle_gemm_f16.argtypes = [vp, vp, vp, vp, ci, ci, ci]
        L.oracle_gemm_awq.argtypes = [vp, vp, vp, vp, vp, vp, ci, ci, ci, ci]
        L.oracle_num_threads.restype = ci
        for n in ("oracle_hadd", "oracle_hsub_ftz", "oracle_hmul_ftz"):
            getattr(L, n).argtypes = [ctypes.c_uint16, ctypes.c_uint16]
            getattr(L, n).restype = ctypes.c_uint16
        L.oracle_f2h.argtypes = [ctypes.c_float]
        L.oracle_f2h.restype = ctypes.c_uint16
        L.oracle_h2f.argtypes = [ctypes.c_uint16]
        L.oracle_h2f.restype = ctypes.c_float
        _lib = L
    return _lib


def _p(a: np.ndarray):
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(ctypes.c_void_p)


def _as_u16(a) -> np.ndarray:
    """fp16 ndarray / torch tensor -> contiguous uint16 bit view."""
    if hasattr(a, "detach"):
        a = a.detach().cpu().contiguous().numpy()
    a = np.ascontiguousarray(a)
    if a.dtype == np.float16:
        a = a.view(np.uint16)
    assert a.dtype == np.uint16, a.dtype
    return a


def _as_np(a, dtype) -> np.ndarray:
    if hasattr(a, "detach"):
        a = a.detach().cpu().contiguous().numpy()
    a = np.ascontiguousarray(a)
    if a.dtype != dtype:
        assert a.dtype.itemsize == np.dtype(dtype).itemsize or a.dtype == np.uint8, (a.dtype, dtype)
        a = a.view(dtype)
    return a


# --------------------------------------------------------------------------------------
# Layout (format.cu restatements)
# --------------------------------------------------------------------------------------

def convert_ours_to_awq(qweight_u8, K: int, N: int) -> np.ndarray:
    """uint8 [N, K/2] -> uint32 [K, N/8]  (format.cu:151-201)."""
    src = _as_np(qweight_u8, np.uint8).reshape(N, K // 2)
    dst = np.empty((K, N // 8), dtype=np.uint32)
    lib().oracle_convert_ours_to_awq(_p(src), _p(dst), K, N)
    return dst


def convert_awq_to_lmdeploy(qweight_awq, K: int, N: int) -> np.ndarray:
    """AWQ uint32 [K, N/8] -> tile-ordered uint32 [K, N/8]  (format.cu:24-71,135-149)."""
    assert K % 32 == 0 and N % 32 == 0
    src = _as_np(qweight_awq, np.uint32).reshape(K, N // 8)
    dst = np.empty((K, N // 8), dtype=np.uint32)
    lib().oracle_convert_awq_to_lmdeploy(_p(src), _p(dst), K, N)
    return dst


def transpose_merge_zeros_scales(zeros, scales, K: int, N: int, g: int) -> np.ndarray:
    """fp16 [N, K/g] x2 -> fp16 bits [K/g, 2N] of (zero+64, scale) pairs  (format.cu:206-239)."""
    z = _as_u16(zeros).reshape(N, K // g)
    s = _as_u16(scales).reshape(N, K // g)
    out = np.empty((K // g, 2 * N), dtype=np.uint16)
    lib().oracle_transpose_merge_zeros_scales(_p(z), _p(s), _p(out), K, N, g)
    return out


def pack(qweight_u8, zeros, scales, K: int, N: int, g: int):
    """The three-op packing flow of quant_lmdeploy (test/nvidia/utils/quant_dequant_nvidia.py:5-32)."""
    zs = transpose_merge_zeros_scales(zeros, scales, K, N, g)
    awq = convert_ours_to_awq(qweight_u8, K, N)
    return convert_awq_to_lmdeploy(awq, K, N), zs


def unpack(qweight, K: int, N: int) -> np.ndarray:
    """tile-ordered uint32 [K, N/8] -> q uint8 [N, K] through the closed-form element address."""
    qw = _as_np(qweight, np.uint32).reshape(-1)
    q = np.empty((N, K), dtype=np.uint8)
    lib().oracle_unpack(_p(qw), _p(q), K, N)
    return q


# --------------------------------------------------------------------------------------
# Dequant + GEMM (common.h / gemm_template.h restatements)
# --------------------------------------------------------------------------------------

def dequant(qweight, zeros_scales, K: int, N: int, g: int) -> np.ndarray:
    """Packed tensors -> dequantised weight, fp16 [N, K] (bit exact: sub.ftz / mul.ftz)."""
    qw = _as_np(qweight, np.uint32).reshape(-1)
    zs = _as_u16(zeros_scales).reshape(-1)
    assert qw.size == K * N // 8 and zs.size == (K // g) * N * 2
    w = np.empty((N, K), dtype=np.uint16)
    lib().oracle_dequant(_p(qw), _p(zs), _p(w), K, N, g)
    return w.view(np.float16)


def dequant_f32(qweight, zeros_scales, K: int, N: int, g: int) -> np.ndarray:
    qw = _as_np(qweight, np.uint32).reshape(-1)
    zs = _as_u16(zeros_scales).reshape(-1)
    w = np.empty((N, K), dtype=np.float32)
    lib().oracle_dequant_f32(_p(qw), _p(zs), _p(w), K, N, g)
    return w


def gemm_f16(x, w, bias=None) -> np.ndarray:
    """fp16 x [M,K] @ fp16 w[N,K]^T with fp32 accumulation, fp16 result (+ fp16 bias add)."""
    xb = _as_u16(x)
    wb = _as_u16(w)
    K = xb.shape[-1]
    xb = xb.reshape(-1, K)
    M, N = xb.shape[0], wb.shape[0]
    assert wb.shape == (N, K)
    bb = None if bias is None else _as_u16(bias).reshape(N)
    out = np.empty((M, N), dtype=np.uint16)
    lib().oracle_gemm_f16(_p(xb), _p(wb), None if bb is None else _p(bb), _p(out), M, N, K)
    return out.view(np.float16)


def gemm_awq(x, qweight, zeros_scales, N: int, K: int, g: int, bias=None) -> np.ndarray:
    """CPU restatement of gemm_awq_ut (+ WALinear's bias add): fp16 [..., K] -> fp16 [M, N]."""
    return gemm_f16(x, dequant(qweight, zeros_scales, K, N, g), bias)


def num_threads() -> int:
    return int(lib().oracle_num_threads())


# --------------------------------------------------------------------------------------
# Quantizer (torch-CPU restatement of the reference's Python; all arithmetic in fp16)
# --------------------------------------------------------------------------------------

def quantize_tensor(w, n_bit: int = 4, q_group_size: int = 128):
    """Per-group asymmetric min-max quantisation along the last dim.

    Restates quantize_tensor, test/nvidia/utils/quant_dequant_nvidia.py:124-148 (the later of
    the two definitions in that file, which is the one in effect):
    scales = clamp(max-min, 1e-5)/15; zeros = clamp(-round(min/scales), 0, 15);
    q = clamp(round(w/scales)+zeros, 0, 15); w_fp16 = (q-zeros)*scales.
    Returns (q [N,K] fp16-valued ints, scales [N,K/g], zeros [N,K/g], w_fp16 [N,K]).
    """
    import torch

    shape = w.shape
    assert shape[-1] % q_group_size == 0
    wg = w.reshape(-1, q_group_size)
    max_val = wg.amax(dim=1, keepdim=True)
    min_val = wg.amin(dim=1, keepdim=True)
    max_int = 2 ** n_bit - 1
    scales = (max_val - min_val).clamp(min=1e-5) / max_int
    zeros = (-torch.round(min_val / scales)).clamp_(0, max_int)
    q = torch.clamp(torch.round(wg / scales) + zeros, 0, max_int)
    w_fp16 = ((q - zeros) * scales).reshape(shape)
    return (q.reshape(shape), scales.reshape(shape[0], -1).contiguous(),
            zeros.reshape(shape[0], -1).contiguous(), w_fp16)


def write_4bit_tensor(q):
    """[N,K] values in 0..15 -> uint8 [N,K/2], byte = q[2i]<<4 | q[2i+1]
    (write_4bit_tensor, test/nvidia/utils/quant_dequant_nvidia.py:79-88)."""
    import torch

    qq = q.to(torch.uint8).reshape(-1, 2)
    return ((qq[:, 0] << 4) + qq[:, 1]).reshape(q.shape[0], q.shape[1] // 2)


def generate_quant(weight_fp16, n_bit: int, group_size: int):
    """generate_quant, test/nvidia/utils/quant_dequant_nvidia.py:103-122:
    returns (qweight uint8 [N,K/2], zeros fp16, scales fp16, w_fp16)."""
    q, scales, zeros, w_fp16 = quantize_tensor(weight_fp16, n_bit, group_size)
    return write_4bit_tensor(q), zeros.half(), scales.half(), w_fp16


def quant_pack(weight_fp16, group_size: int = 128):
    """weight fp16 [N,K] -> (qweight uint32 [K,N/8], zeros_scales uint16 [K/g,2N], w_fp16 torch)."""
    N, K = weight_fp16.shape
    qw8, zeros, scales, w_fp16 = generate_quant(weight_fp16, 4, group_size)
    qweight, zs = pack(qw8, zeros, scales, K, N, group_size)
    return qweight, zs, w_fp16


def decode_attention(q, k_new, v_new, k_cache, v_cache, pos: int, scale: float, cos=None, sin=None):
    """Float64 restatement of one decode step of dense attention as the reference's OPT layer does it with torch
    ops (test/nvidia/module/opt/modeling_opt_ours.py: new key/value appended to the cache :249-250, q.K^T :306,
    softmax over the positions seen so far, P.V :456), plus the "rotate half" rotary embedding of the LLaMA-shaped
    stack.  "Parity unpinned": the reference holds no golden vectors for attention; this is the mathematical
    definition, compared with a stated floating-point tolerance.

    q, k_new, v_new [B, H, D]; caches [B, H, L, D] (rows < pos are the past); cos/sin [D] of position `pos`.
    Returns (out [B, H, D] float64, k_row fp16 [B, H, D] as stored in the cache, v_row fp16)."""
    q = np.asarray(q, dtype=np.float64)
    k = np.asarray(k_new, dtype=np.float64)
    v = np.asarray(v_new, dtype=np.float64)
    if cos is not None:
        d = q.shape[-1] // 2
        c, s = np.asarray(cos, dtype=np.float64), np.asarray(sin, dtype=np.float64)

        def rot(x):
            return x * c + np.concatenate((-x[..., d:], x[..., :d]), axis=-1) * s
        q, k = rot(q), rot(k)
    k_row, v_row = k.astype(np.float16), v.astype(np.float16)
    keys = np.concatenate((np.asarray(k_cache, dtype=np.float64)[:, :, :pos], k_row.astype(np.float64)[:, :, None]), axis=2)
    vals = np.concatenate((np.asarray(v_cache, dtype=np.float64)[:, :, :pos], v_row.astype(np.float64)[:, :, None]), axis=2)
    scores = np.einsum("bhd,bhtd->bht", q, keys) * scale
    scores -= scores.max(axis=-1, keepdims=True)
    p = np.exp(scores)
    p /= p.sum(axis=-1, keepdims=True)
    return np.einsum("bht,bhtd->bhd", p, vals), k_row, v_row
