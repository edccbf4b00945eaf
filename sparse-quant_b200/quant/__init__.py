"""`quant` — drop-in for the reference's CUDA extension of the same name, on B200.

The reference builds a pybind11 module `quant` (quantization/nvidia/kernel/pybind.cpp:7-12)
with four functions; this package exposes the same four names with the same positional
arguments, tensor formats and error behaviour (RuntimeError on bad arguments, as TORCH_CHECK
raises in kernel/utils.h:10-16), plus `dequant` (named after the op of the reference's
sibling backend, quantization/tianshu/backend/pybind.cpp:12).

The work is done by hand-written sm_100a kernels behind a C ABI (include/w4a16_b200.h,
libw4a16_b200.so next to this file) called through ctypes; torch only provides device
memory and the current stream.  There is no CPU path and no fallback: importing works
anywhere (so the host logic can be tested), calling a function without the built library
or without a B200 raises.
"""
from __future__ import annotations

import ctypes
import os

import torch

__all__ = [
    "gemm_awq_ut", "transpose_merge_zeros_scales", "convert_ours_to_awq", "convert_awq_to_lmdeploy",
    "dequant", "quantize_pack", "gemm_awq_bias", "library_path", "load_library", "launch_count",
]

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_NAME = "libw4a16_b200.so"
_lib = None

ALGO_AUTO, ALGO_SKINNY, ALGO_TC = 0, 1, 2

# every symbol include/w4a16_b200.h declares: name -> (restype, argtypes)
_vp, _ci, _sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t
C_ABI = {
    "w4a16_status_str": (ctypes.c_char_p, [_ci]),
    "w4a16_last_cuda_error": (_ci, []),
    "w4a16_gemm": (_ci, [_vp, _vp, _vp, _vp, _vp, _ci, _ci, _ci, _ci, _vp, _sz, _vp]),
    "w4a16_gemm_algo": (_ci, [_vp, _vp, _vp, _vp, _vp, _ci, _ci, _ci, _ci, _vp, _sz, _vp, _ci]),
    "w4a16_gemm_ex": (_ci, [_vp, _vp, _vp, _vp, _vp, _ci, _ci, _ci, _ci, _vp, _sz, _vp, _ci, ctypes.c_uint]),
    "w4a16_gemm_fused": (_ci, [_vp, _vp, _vp, _vp, _vp, _vp, _ci, _ci, _ci, _ci, _vp, _sz, _vp, _ci, ctypes.c_uint]),
    "w4a16_gemm_prenorm": (_ci, [_vp, _vp, _vp, _vp, ctypes.c_float, _ci, _vp, _vp, _vp, _vp, _ci, _ci, _ci, _ci, _vp, ctypes.c_uint]),
    "w4a16_gemm_residual_stats": (_ci, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _ci, _ci, _ci, _ci, _vp, ctypes.c_uint]),
    "w4a16_row_stats_bytes": (_sz, [_ci]),
    "w4a16_workspace_bytes": (_sz, [_ci, _ci, _ci, _ci]),
    "w4a16_exchange_bytes": (_sz, [_ci, _sz]),
    "w4a16_exchange_alloc": (_ci, [_ci, _sz, ctypes.POINTER(_vp)]),
    "w4a16_exchange_free": (_ci, [_vp]),
    "w4a16_exchange_export": (_ci, [_vp, _vp]),
    "w4a16_exchange_open": (_ci, [_vp, ctypes.POINTER(_vp)]),
    "w4a16_exchange_close": (_ci, [_vp]),
    "w4a16_exchange_status": (_ci, [_vp, ctypes.POINTER(ctypes.c_uint), ctypes.POINTER(_ci)]),
    "w4a16_exchange_allgather": (_ci, [_vp, _vp, _ci, ctypes.POINTER(_vp), _ci, _ci, _sz, _vp]),
    "w4a16_gemm_allreduce": (_ci, [_vp, _vp, _vp, _vp, _vp, _ci, _ci, _ci, _ci, _ci, ctypes.POINTER(_vp), _ci, _ci, _sz,
                                   _vp, ctypes.c_uint]),
    "w4a16_allreduce_supported": (_ci, [_ci, _ci, _ci, _ci, _ci, _ci]),
    "w4a16_gemm_allreduce_residual": (_ci, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _ci, _ci, _ci, _ci, _ci, ctypes.POINTER(_vp), _ci,
                                            _ci, _sz, _vp, ctypes.c_uint]),
    "w4a16_decode_attention": (_ci, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _ci, _ci, _ci, _ci, _ci, ctypes.c_float, _vp]),
    "w4a16_tune_attention": (None, [_ci]),
    "w4a16_tune_aux_launch": (None, [_ci]),
    "w4a16_add_norm": (_ci, [_vp, _vp, _vp, _vp, _vp, _vp, _ci, _ci, ctypes.c_float, _ci, _vp]),
    "w4a16_silu_mul": (_ci, [_vp, _vp, _ci, _ci, _vp]),
    "w4a16_gemm_static_scratch": (_ci, [_vp, _vp, _vp, _vp, _vp, _ci, _ci, _ci, _ci, _vp]),
    "w4a16_static_scratch_error_flag": (_ci, [ctypes.POINTER(_ci)]),
    "w4a16_dequant": (_ci, [_vp, _vp, _vp, _ci, _ci, _ci, _vp]),
    "w4a16_transpose_merge_zeros_scales": (_ci, [_vp, _vp, _vp, _ci, _ci, _ci, _vp]),
    "w4a16_convert_ours_to_awq": (_ci, [_vp, _vp, _ci, _ci, _vp]),
    "w4a16_convert_awq_to_lmdeploy": (_ci, [_vp, _vp, _ci, _ci, _vp]),
    "w4a16_quantize_pack": (_ci, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _ci, _ci, _ci, _vp]),
    "w4a16_gemm_host": (_ci, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _ci, _ci, _ci, _ci, _vp, _sz, _vp]),
    "w4a16_gemm_host_async": (_ci, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _ci, _ci, _ci, _ci, _vp, _sz, _vp]),
    "w4a16_launch_count": (ctypes.c_ulonglong, []),
    "w4a16_version": (_ci, []),
    "w4a16_device_error_flag": (_ci, [ctypes.POINTER(_ci)]),
    "w4a16_debug_tmem_layout": (_ci, [_vp, _vp]),
    "w4a16_debug_skinny_timeline": (None, [_vp]),
    "w4a16_tune_skinny": (None, [_ci, _ci]),
    "w4a16_tune_tc": (None, [_ci, _ci]),
    "w4a16_tune_decode": (None, [_ci, _ci, _ci, _ci]),
    "w4a16_tune_decode_prefetch": (None, [_ci]),
    "w4a16_debug_decode_plan": (_ci, [_ci, _ci, _ci, _ci, ctypes.POINTER(_ci)]),
    "w4a16_device_error_clear": (_ci, []),
    "w4a16_exchange_reset": (_ci, [_vp]),
    "w4a16_tune_exchange_wait": (None, [ctypes.c_uint]),
}


def library_path() -> str:
    return os.path.join(_HERE, _LIB_NAME)


def load_library() -> ctypes.CDLL:
    """Load the C-ABI library (built by sparse-quant_b200/build.py).  Raises if it is missing."""
    global _lib
    if _lib is None:
        path = library_path()
        if not os.path.exists(path):
            raise RuntimeError(
                f"{_LIB_NAME} is not built (expected at {path}); run `python sparse-quant_b200/build.py`. "
                "There is no CPU or PyTorch fallback for the W4A16 kernels.")
        lib = ctypes.CDLL(path)
        for name, (res, args) in C_ABI.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def _check(status: int, what: str) -> None:
    if status != 0:
        lib = load_library()
        msg = lib.w4a16_status_str(status).decode()
        extra = f" (cudaError {lib.w4a16_last_cuda_error()})" if status == 7 else ""
        raise RuntimeError(f"{what}: {msg}{extra}")


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def _check_tensor(t, name, *, dtype=None, dims=None):
    _need(isinstance(t, torch.Tensor), f"{name} must be a torch.Tensor")
    _need(t.is_cuda, f"Tensor {name} must be on CUDA")
    _need(t.is_contiguous(), f"Tensor {name} must be contiguous")
    if dtype is not None:
        _need(t.dtype == dtype, f"Tensor {name} must have dtype ({dtype})")
    if dims is not None:
        _need(t.dim() == dims, f"Tensor {name} must have dimension number ({dims})")


def launch_count() -> int:
    """Kernels launched by the library in this process so far."""
    return int(load_library().w4a16_launch_count())


FLAG_STATIC_WEIGHTS = 1
FLAG_RELU = 2
FLAG_SILU_MUL = 4


def prenorm_supported(tokens: int, K: int) -> bool:
    """Whether w4a16_gemm_prenorm takes this input (see include/w4a16_b200.h)."""
    return 0 < tokens <= 16 and K % 8 == 0 and K <= 8192


def row_stats_supported(tokens: int) -> bool:
    """Whether w4a16_gemm_residual_stats / w4a16_gemm_allreduce_residual write row statistics for this many tokens."""
    return 0 < tokens <= 16


def row_stats_buffer(N: int, device):
    """A buffer for the row statistics a GEMV with N out-features leaves for the GEMV that normalises its output."""
    return torch.zeros(load_library().w4a16_row_stats_bytes(int(N)) // 4, dtype=torch.float32, device=device)


def gemm_awq_bias(I, W, W_zeros_scales, bias, N: int, group_size: int, algo: int = ALGO_AUTO, out=None,
                  static_weights: bool = False, relu: bool = False, residual=None, silu_mul: bool = False,
                  pre_norm=None, stats_out=None):
    """gemm_awq_ut with the fp16 bias add of WALinear.forward fused into the kernel epilogue.

    I fp16 [b, s, K] (CUDA, contiguous); W int32 [K, N/8] tile-ordered; W_zeros_scales fp16
    [K/g, 2N]; bias fp16 with N elements or None.  Returns fp16 [b, s, N].
    static_weights=True passes W4A16_FLAG_STATIC_WEIGHTS (see include/w4a16_b200.h): only for weights
    that were written before anything still in flight on the current stream was enqueued.
    relu=True passes W4A16_FLAG_RELU: max(., 0) applied after the bias add.
    residual (fp16 [b, s, N]) is added to the output in the kernel epilogue; silu_mul=True passes
    W4A16_FLAG_SILU_MUL (gate / up tiles interleaved, see w4a16_gemm_fused): returns fp16 [b, s, N/2].
    pre_norm = (weight, bias or None, eps, rms, stats): the linear is applied to LayerNorm / RMSNorm of I; `stats` is the
    row_stats_buffer the GEMV that produced I filled (stats_out=...), or None: the normalisation then runs as its own
    launch.  stats_out: leave the row statistics of this call's output there (up to 16 tokens; ignored beyond).
    """
    _check_tensor(I, "I", dtype=torch.float16, dims=3)
    _check_tensor(W, "W", dims=2)
    _check_tensor(W_zeros_scales, "W_zeros_scales", dtype=torch.float16, dims=2)
    b, s, K = I.shape
    N = int(N)
    group_size = int(group_size)
    _need(W.device == I.device and W_zeros_scales.device == I.device, "all tensors must be on the same device")
    _need(group_size > 0 and N > 0, "unsupported group size" if group_size <= 0 else "N must be positive")
    _need(W.numel() * W.element_size() * 2 == K * N, f"Tensor W must hold K*N/2 = {K * N // 2} bytes of packed int4")
    _need(K % group_size == 0 and W_zeros_scales.numel() == (K // group_size) * N * 2,
          "Tensor W_zeros_scales must have K/group_size * 2N elements")
    if bias is not None:
        _check_tensor(bias, "bias", dtype=torch.float16)
        _need(bias.numel() == N and bias.device == I.device, "Tensor bias must have N elements on the same device")
    n_out = N // 2 if silu_mul else N
    if residual is not None:
        _check_tensor(residual, "residual", dtype=torch.float16)
        _need(residual.numel() == b * s * N and residual.device == I.device, "Tensor residual must have b*s*N elements")
    if out is None:
        out = torch.empty((b, s, n_out), dtype=torch.float16, device=I.device)
    else:
        _check_tensor(out, "O", dtype=torch.float16, dims=3)
        _need(tuple(out.shape) == (b, s, n_out) and out.device == I.device, "Tensor O must have shape [b, s, N]")
    lib = load_library()
    tokens = b * s
    if pre_norm is not None:
        # (weight, bias or None, eps, rms): I is the un-normalised input; the normalisation runs inside the decode
        # kernel while it stages its activations (w4a16_gemm_prenorm), or as its own launch where that has no room
        nw, nb, eps, rms, stats = pre_norm if len(pre_norm) == 5 else (*pre_norm, None)
        _check_tensor(nw, "norm weight", dtype=torch.float16)
        _need(nw.numel() == K and nw.device == I.device, "norm weight must have K elements on the same device")
        if nb is not None:
            _check_tensor(nb, "norm bias", dtype=torch.float16)
            _need(nb.numel() == K and nb.device == I.device, "norm bias must have K elements on the same device")
        if stats is not None and residual is None and algo == ALGO_AUTO and prenorm_supported(tokens, K):
            with torch.cuda.device(I.device):
                st = lib.w4a16_gemm_prenorm(I.data_ptr(), stats.data_ptr(), nw.data_ptr(),
                                            nb.data_ptr() if (nb is not None and not rms) else None,
                                            float(eps), int(bool(rms)), W.data_ptr(), W_zeros_scales.data_ptr(),
                                            bias.data_ptr() if bias is not None else None, out.data_ptr(), tokens, N, K,
                                            group_size, _stream(I),
                                            (FLAG_STATIC_WEIGHTS if static_weights else 0) | (FLAG_RELU if relu else 0) |
                                            (FLAG_SILU_MUL if silu_mul else 0))
            _check(st, "gemm_awq_ut")
            return out
        I = add_norm(I, None, nw, nb, eps, rms)[1]
    if stats_out is not None and not silu_mul and algo == ALGO_AUTO and row_stats_supported(tokens):
        with torch.cuda.device(I.device):
            st = lib.w4a16_gemm_residual_stats(I.data_ptr(), W.data_ptr(), W_zeros_scales.data_ptr(),
                                               bias.data_ptr() if bias is not None else None,
                                               residual.data_ptr() if residual is not None else None, out.data_ptr(),
                                               stats_out.data_ptr(), tokens, N, K, group_size, _stream(I),
                                               (FLAG_STATIC_WEIGHTS if static_weights else 0) | (FLAG_RELU if relu else 0))
        _check(st, "gemm_awq_ut")
        return out
    with torch.cuda.device(I.device):
        ws_bytes = lib.w4a16_workspace_bytes(tokens, N, K, group_size)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=I.device) if ws_bytes else None
        st = lib.w4a16_gemm_fused(I.data_ptr(), W.data_ptr(), W_zeros_scales.data_ptr(),
                                  bias.data_ptr() if bias is not None else None,
                                  residual.data_ptr() if residual is not None else None, out.data_ptr(),
                                  tokens, N, K, group_size,
                                  ws.data_ptr() if ws is not None else None, ws_bytes, _stream(I), int(algo),
                                  (FLAG_STATIC_WEIGHTS if static_weights else 0) | (FLAG_RELU if relu else 0) |
                                  (FLAG_SILU_MUL if silu_mul else 0))
    _check(st, "gemm_awq_ut")
    return out


def gemm_awq_allreduce(I, W, W_zeros_scales, bias, N: int, group_size: int, k_config: int, buffers, world: int,
                       rank: int, capacity: int, out=None, static_weights: bool = False, residual=None, stats_out=None):
    """Row-parallel linear for decode: this rank's K shard times its slice of the activations, summed over the
    ranks inside the kernel through peer memory (see w4a16_gemm_allreduce in include/w4a16_b200.h).

    I fp16 [b, s, K_shard] with b*s <= 32; `buffers` is a ctypes array of `world` device pointers (every rank's
    exchange buffer, own included); `bias` (N elements or None) must be the same on all ranks and is added once.
    `residual` (fp16 [b, s, N], the same on all ranks, or None) is added once to the summed output.
    Returns fp16 [b, s, N], identical on every rank.
    """
    _check_tensor(I, "I", dtype=torch.float16, dims=3)
    _check_tensor(W, "W", dims=2)
    _check_tensor(W_zeros_scales, "W_zeros_scales", dtype=torch.float16, dims=2)
    b, s, K = I.shape
    N, group_size = int(N), int(group_size)
    _need(b * s <= 32, "gemm_awq_allreduce handles at most 32 tokens")
    _need(W.numel() * W.element_size() * 2 == K * N, f"Tensor W must hold K*N/2 = {K * N // 2} bytes of packed int4")
    _need(group_size > 0 and K % group_size == 0 and W_zeros_scales.numel() == (K // group_size) * N * 2,
          "Tensor W_zeros_scales must have K/group_size * 2N elements")
    if bias is not None:
        _check_tensor(bias, "bias", dtype=torch.float16)
        _need(bias.numel() == N, "Tensor bias must have N elements")
    if residual is not None:
        _check_tensor(residual, "residual", dtype=torch.float16)
        _need(residual.numel() == b * s * N and residual.device == I.device, "Tensor residual must have b*s*N elements")
    if out is None:
        out = torch.empty((b, s, N), dtype=torch.float16, device=I.device)
    lib = load_library()
    with torch.cuda.device(I.device):
        st = lib.w4a16_gemm_allreduce_residual(I.data_ptr(), W.data_ptr(), W_zeros_scales.data_ptr(),
                                               bias.data_ptr() if bias is not None else None,
                                               residual.data_ptr() if residual is not None else None, out.data_ptr(),
                                               stats_out.data_ptr() if (stats_out is not None and b * s <= 16) else None,
                                               b * s, N, K, group_size, int(k_config), buffers, int(world), int(rank),
                                               int(capacity), _stream(I), FLAG_STATIC_WEIGHTS if static_weights else 0)
    _check(st, "gemm_awq_allreduce")
    return out


def add_norm(x, delta, weight, bias, eps: float, rms: bool):
    """(x + delta, norm(x + delta)) in one launch (see w4a16_add_norm in include/w4a16_b200.h); delta None: (x, norm(x)).
    x, delta fp16 [..., cols] contiguous; LayerNorm (rms=False, fp16 weight/bias) or RMSNorm (rms=True)."""
    _check_tensor(x, "x", dtype=torch.float16)
    _check_tensor(weight, "weight", dtype=torch.float16)
    cols = x.shape[-1]
    rows = x.numel() // cols
    _need(weight.numel() == cols, "weight must have one element per column")
    if delta is not None:
        _check_tensor(delta, "delta", dtype=torch.float16)
        _need(delta.shape == x.shape, "delta must have the shape of x")
    if bias is not None:
        _check_tensor(bias, "bias", dtype=torch.float16)
    s = torch.empty_like(x) if delta is not None else x
    h = torch.empty_like(x)
    lib = load_library()
    with torch.cuda.device(x.device):
        st = lib.w4a16_add_norm(x.data_ptr(), delta.data_ptr() if delta is not None else None,
                                s.data_ptr() if delta is not None else None, h.data_ptr(), weight.data_ptr(),
                                bias.data_ptr() if (bias is not None and not rms) else None, rows, cols, float(eps), int(bool(rms)),
                                _stream(x))
    _check(st, "add_norm")
    return s, h


def silu_mul(gate_up):
    """fp16 [..., 2n] (gate | up) -> silu(gate) * up, fp16 [..., n] (see w4a16_silu_mul in include/w4a16_b200.h)."""
    _check_tensor(gate_up, "gate_up", dtype=torch.float16)
    n = gate_up.shape[-1] // 2
    rows = gate_up.numel() // (2 * n)
    out = torch.empty(tuple(gate_up.shape[:-1]) + (n,), dtype=torch.float16, device=gate_up.device)
    lib = load_library()
    with torch.cuda.device(gate_up.device):
        _check(lib.w4a16_silu_mul(gate_up.data_ptr(), out.data_ptr(), rows, n, _stream(gate_up)), "silu_mul")
    return out


def decode_attention(qkv, k_cache, v_cache, pos, heads: int, rope=None, scale=None, out=None):
    """One decode step of attention over a static cache (see w4a16_decode_attention in include/w4a16_b200.h).

    qkv fp16 [B, >= 3*heads*D] (q | k | v of the new token), k_cache / v_cache fp16 [B, heads, max_len, D]
    (contiguous; updated in place at row `pos`), pos int64 CUDA tensor with one element, rope = (cos, sin) fp16
    [positions, D] tables or None.  Returns fp16 [B, heads*D]."""
    _check_tensor(qkv, "qkv", dtype=torch.float16, dims=2)
    _check_tensor(k_cache, "k_cache", dtype=torch.float16, dims=4)
    _check_tensor(v_cache, "v_cache", dtype=torch.float16, dims=4)
    B, H, max_len, D = k_cache.shape
    _need(H == int(heads) and tuple(v_cache.shape) == tuple(k_cache.shape), "cache shape must be [B, heads, max_len, D]")
    _need(qkv.shape[0] == B and qkv.shape[1] >= 3 * H * D, "qkv must be [B, >= 3*heads*D]")
    _need(pos.is_cuda and pos.dtype == torch.int64 and pos.numel() == 1, "pos must be one int64 on the device")
    cos = sin = None
    if rope is not None:
        cos, sin = rope
        _check_tensor(cos, "rope cos", dtype=torch.float16, dims=2)
        _check_tensor(sin, "rope sin", dtype=torch.float16, dims=2)
        _need(cos.shape[1] == D and sin.shape == cos.shape and cos.shape[0] >= max_len, "rope tables must be [>= max_len, D]")
    if out is None:
        out = torch.empty((B, H * D), dtype=torch.float16, device=qkv.device)
    lib = load_library()
    with torch.cuda.device(qkv.device):
        st = lib.w4a16_decode_attention(qkv.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), pos.data_ptr(),
                                        cos.data_ptr() if cos is not None else None, sin.data_ptr() if sin is not None else None,
                                        B, H, D, max_len, qkv.stride(0), float(D ** -0.5 if scale is None else scale), _stream(qkv))
    _check(st, "decode_attention")
    return out


def gemm_awq_ut(I, W, W_zeros_scales, M: int, N: int, K: int, group_size: int):
    """O[b, s, :] = I[b, s, :] @ dequant(W, W_zeros_scales)^T, fp16.

    Same signature as the reference's gemm_awq_ut (kernel/gemm_quant.h:15-17,
    kernel/gemm_quant.cu:98-122).  As there, `M` and `K` are accepted and ignored: the token
    count and K come from `I` (gemm_quant.cu:85-87); `I` must be 3-D.  Launches on torch's
    current stream (the reference uses the legacy default stream).
    """
    return gemm_awq_bias(I, W, W_zeros_scales, None, N, group_size)


def transpose_merge_zeros_scales(zeros, scales, zeros_scales, in_features: int, out_features: int, group_size: int):
    """zeros_scales[k/g, 2n:2n+2] = (zeros[n, k/g] + 64, scales[n, k/g]); in place, returns None.
    Reference: kernel/gemm_s4_f16/format.cu:206-239."""
    _check_tensor(zeros, "zeros", dtype=torch.float16)
    _check_tensor(scales, "scales", dtype=torch.float16)
    _check_tensor(zeros_scales, "zeros_scales", dtype=torch.float16)
    _need(int(group_size) > 0 and in_features % int(group_size) == 0, "in_features must be a multiple of group_size")
    groups = in_features // int(group_size)
    _need(zeros.numel() == out_features * groups and scales.numel() == out_features * groups,
          "zeros/scales must have out_features * in_features/group_size elements")
    _need(zeros_scales.numel() == groups * out_features * 2, "zeros_scales must have in_features/group_size * 2*out_features elements")
    with torch.cuda.device(zeros.device):
        st = load_library().w4a16_transpose_merge_zeros_scales(
            zeros.data_ptr(), scales.data_ptr(), zeros_scales.data_ptr(), int(in_features), int(out_features),
            int(group_size), _stream(zeros))
    _check(st, "transpose_merge_zeros_scales")


def convert_ours_to_awq(qweight_src, qweight_dst, in_features: int, out_features: int):
    """uint8 [N, K/2] -> AWQ-ordered words written into qweight_dst (uint8 [K, N/2], i.e. uint32
    [K, N/8]); in place, returns None.  Reference: kernel/gemm_s4_f16/format.cu:151-201."""
    _check_tensor(qweight_src, "qweight_src", dtype=torch.uint8)
    _check_tensor(qweight_dst, "qweight_dst")
    _need(qweight_src.numel() == in_features * out_features // 2, "qweight_src must have out_features * in_features/2 bytes")
    _need(qweight_dst.numel() * qweight_dst.element_size() == in_features * out_features // 2,
          "qweight_dst must have in_features * out_features/2 bytes")
    with torch.cuda.device(qweight_src.device):
        st = load_library().w4a16_convert_ours_to_awq(qweight_src.data_ptr(), qweight_dst.data_ptr(),
                                                      int(in_features), int(out_features), _stream(qweight_src))
    _check(st, "convert_ours_to_awq")


def convert_awq_to_lmdeploy(qweight, qweight_dst, in_features: int, out_features: int):
    """AWQ words -> tile-ordered int32 [K, N/8] (the `weight` buffer the GEMM reads); in place,
    returns None.  Reference: kernel/gemm_s4_f16/format.cu:135-149,24-71."""
    _check_tensor(qweight, "qweight")
    _check_tensor(qweight_dst, "qweight_dst")
    nbytes = in_features * out_features // 2
    _need(qweight.numel() * qweight.element_size() == nbytes, "qweight must have in_features * out_features/2 bytes")
    _need(qweight_dst.numel() * qweight_dst.element_size() == nbytes, "qweight_dst must have in_features * out_features/2 bytes")
    with torch.cuda.device(qweight.device):
        st = load_library().w4a16_convert_awq_to_lmdeploy(qweight.data_ptr(), qweight_dst.data_ptr(),
                                                          int(in_features), int(out_features), _stream(qweight))
    _check(st, "convert_awq_to_lmdeploy")


def quantize_pack(weight, in_features: int, out_features: int, group_size: int, parts: bool = False):
    """fp16 weight [N, K] (CUDA) -> (weight int32 [K, N/8] tile-ordered, zeros_scales fp16 [K/g, 2N], w_fp16 [N, K])
    in one kernel, bit-identical to the reference's quantise-and-pack flow (see w4a16_quantize_pack in
    include/w4a16_b200.h).  parts=True also returns (qweight_ours uint8 [N, K/2], zeros, scales fp16 [N, K/g]), the
    intermediate tensors of the reference's generate_quant."""
    _check_tensor(weight, "weight", dtype=torch.float16, dims=2)
    N, K, g = int(out_features), int(in_features), int(group_size)
    _need(tuple(weight.shape) == (N, K), "Tensor weight must have shape [out_features, in_features]")
    dev = weight.device
    qweight = torch.empty((K, N // 8), dtype=torch.int32, device=dev)
    zeros_scales = torch.empty((K // g if g > 0 else 0, 2 * N), dtype=torch.float16, device=dev)
    w_fp16 = torch.empty((N, K), dtype=torch.float16, device=dev)
    ours = zeros = scales = None
    if parts:
        ours = torch.empty((N, K // 2), dtype=torch.uint8, device=dev)
        zeros = torch.empty((N, K // g), dtype=torch.float16, device=dev)
        scales = torch.empty((N, K // g), dtype=torch.float16, device=dev)
    with torch.cuda.device(dev):
        st = load_library().w4a16_quantize_pack(
            weight.data_ptr(), qweight.data_ptr(), zeros_scales.data_ptr(), w_fp16.data_ptr(),
            zeros.data_ptr() if parts else None, scales.data_ptr() if parts else None, ours.data_ptr() if parts else None,
            K, N, g, _stream(weight))
    _check(st, "quantize_pack")
    return (qweight, zeros_scales, w_fp16, ours, zeros, scales) if parts else (qweight, zeros_scales, w_fp16)


def dequant(W, W_zeros_scales, N: int, K: int, group_size: int):
    """Packed tensors -> fp16 [N, K] weight, bit-exact with the reference's in-kernel dequantisation
    (kernel/gemm_s4_f16/common.h:114-153,210-225)."""
    _check_tensor(W, "W", dims=2)
    _check_tensor(W_zeros_scales, "W_zeros_scales", dtype=torch.float16, dims=2)
    _need(W.numel() * W.element_size() * 2 == K * N, "Tensor W must hold K*N/2 bytes of packed int4")
    _need(int(group_size) > 0 and K % int(group_size) == 0 and
          W_zeros_scales.numel() == (K // int(group_size)) * N * 2, "Tensor W_zeros_scales must have K/group_size * 2N elements")
    out = torch.empty((N, K), dtype=torch.float16, device=W.device)
    with torch.cuda.device(W.device):
        st = load_library().w4a16_dequant(W.data_ptr(), W_zeros_scales.data_ptr(), out.data_ptr(), int(N), int(K),
                                          int(group_size), _stream(W))
    _check(st, "dequant")
    return out
