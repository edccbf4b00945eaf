"""The give-up paths of the device-side waits, executed on one GPU without faulting, trapping or hanging it.

A kernel that waits for a peer polls with a time limit; when the limit runs out it records why, marks the exchange
buffer and RETURNS, so the context stays usable.  Here the limit is made to run out on purpose: a two-rank exchange
whose second rank never shows up (its buffer is a second allocation on this GPU that nobody writes), with the limit
turned down to a few milliseconds.  Checked: the device error word (2), which rank was late, that the next call does
not wait again, that both marks can be cleared, and that the GPU still answers a plain GEMV afterwards.  The decode
attention kernel's refusal of a position outside the cache (error word 3) is checked the same way."""
import ctypes
import time

import numpy as np
import pytest
import torch

import oracle
from helpers import check_gemm_tolerance, make_packed, make_x, to_dev

pytestmark = pytest.mark.gpu


def _flag(lib):
    f = ctypes.c_int(-1)
    assert lib.w4a16_device_error_flag(ctypes.byref(f)) == 0
    return f.value


@pytest.fixture()
def two_rank_buffers():
    import quant
    lib = quant.load_library()
    assert _flag(lib) == 0, "an earlier test left the device error word set"
    cap = 32 * 256
    bufs = (ctypes.c_void_p * 2)()
    for r in range(2):
        b = ctypes.c_void_p()
        assert lib.w4a16_exchange_alloc(2, cap, ctypes.byref(b)) == 0
        bufs[r] = b.value
    lib.w4a16_tune_exchange_wait(5)                       # milliseconds
    try:
        yield lib, bufs, cap
    finally:
        lib.w4a16_tune_exchange_wait(0)
        lib.w4a16_device_error_clear()
        for r in range(2):
            lib.w4a16_exchange_free(ctypes.c_void_p(bufs[r]))


@pytest.mark.parametrize("tokens", [4, 24])               # 8-warp kernel, 16-warp kernel
def test_exchange_wait_runs_out_and_the_kernel_returns(two_rank_buffers, tokens):
    lib, bufs, cap = two_rank_buffers
    N, K, g = 256, 512, 128
    p = make_packed(N, K, g, seed=31)
    qw, zs = to_dev(p)
    x = make_x(tokens, K).cuda()[0].contiguous()
    out = torch.zeros(tokens, N, dtype=torch.float16, device="cuda")
    sp = torch.cuda.current_stream().cuda_stream

    def call():
        return lib.w4a16_gemm_allreduce(x.data_ptr(), qw.data_ptr(), zs.data_ptr(), None, out.data_ptr(), tokens, N, K, g, K,
                                        bufs, 2, 0, cap, sp, 0)

    t0 = time.perf_counter()
    assert call() == 0
    torch.cuda.synchronize()                                # returns: the wait is bounded
    first = time.perf_counter() - t0
    assert first < 2.0
    assert _flag(lib) == 2                                  # "a wait for a peer in the exchange gave up"
    epoch, err = ctypes.c_uint(0), ctypes.c_int(0)
    assert lib.w4a16_exchange_status(ctypes.c_void_p(bufs[0]), ctypes.byref(epoch), ctypes.byref(err)) == 0
    assert err.value == 2 and epoch.value == 1              # 1 + the late rank; the call still completed its epoch
    # the buffer stays marked: later calls do not wait for the missing rank again
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    assert call() == 0
    e1.record()
    torch.cuda.synchronize()
    assert e0.elapsed_time(e1) < 2.0                        # milliseconds; the limit alone is 5
    # both marks can be cleared, after which a call waits (and gives up) again
    assert lib.w4a16_device_error_clear() == 0 and _flag(lib) == 0
    assert lib.w4a16_exchange_reset(ctypes.c_void_p(bufs[0])) == 0
    assert lib.w4a16_exchange_status(ctypes.c_void_p(bufs[0]), ctypes.byref(epoch), ctypes.byref(err)) == 0 and err.value == 0
    assert call() == 0
    torch.cuda.synchronize()
    assert _flag(lib) == 2
    assert lib.w4a16_device_error_clear() == 0
    # the GPU still answers: a plain GEMV on the same tensors matches the oracle
    import quant
    y = quant.gemm_awq_bias(x.unsqueeze(0), qw, zs, None, N, g)
    torch.cuda.synchronize()
    ref = oracle.gemm_f16(x.cpu().unsqueeze(0), p["w_deq"]).astype(np.float32)
    check_gemm_tolerance(y[0], ref, x, p["w_deq"], K)
    assert _flag(lib) == 0


def test_allgather_wait_runs_out(two_rank_buffers):
    lib, bufs, cap = two_rank_buffers
    words = 16
    src = torch.arange(words, dtype=torch.int32, device="cuda")
    dst = torch.full((2 * words,), -1, dtype=torch.int32, device="cuda")
    assert lib.w4a16_exchange_allgather(src.data_ptr(), dst.data_ptr(), words, bufs, 2, 0, cap,
                                        torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    assert _flag(lib) == 2
    assert torch.equal(dst[:words], src)                    # this rank's own words did arrive
    err = ctypes.c_int(0)
    assert lib.w4a16_exchange_status(ctypes.c_void_p(bufs[0]), None, ctypes.byref(err)) == 0 and err.value == 2


def test_attention_refuses_a_position_outside_the_cache():
    import quant
    lib = quant.load_library()
    assert _flag(lib) == 0
    B, H, D, L = 2, 2, 64, 16
    gen = torch.Generator().manual_seed(3)
    qkv = torch.randn(B, 3 * H * D, generator=gen).half().cuda()
    kc = torch.randn(B, H, L, D, generator=gen).half().cuda()
    vc = torch.randn(B, H, L, D, generator=gen).half().cuda()
    kc0, vc0 = kc.clone(), vc.clone()
    out = torch.full((B, H * D), 7.0, dtype=torch.float16, device="cuda")
    try:
        quant.decode_attention(qkv, kc, vc, torch.tensor([L], device="cuda"), H, out=out)     # one past the end
        torch.cuda.synchronize()
        assert _flag(lib) == 3
        assert torch.equal(kc, kc0) and torch.equal(vc, vc0) and bool((out == 7.0).all())     # nothing was written
    finally:
        assert lib.w4a16_device_error_clear() == 0
    quant.decode_attention(qkv, kc, vc, torch.tensor([L - 1], device="cuda"), H, out=out)     # still usable
    torch.cuda.synchronize()
    assert _flag(lib) == 0 and not bool((out == 7.0).all())
