"""The allocation-free entry point (w4a16_gemm_static_scratch).

Who needs it: code that may not call cudaMalloc while it runs - work issued during stream capture,
plug-ins inside a runtime that owns the device allocator, services whose memory budget is fixed at
start-up.  The split-K tcgen05 GEMM normally takes its scratch (fp32 partial tiles, arrival counters)
from a caller-provided workspace and its error word from a one-time cudaMalloc; this entry point keeps
all of that in a device array that is part of the library image.  Checked here, through the C ABI: its
output against the regular entry point and against the CPU oracle on two calls in a row (the array is shared
and keeps the previous call's contents), its size limit, and that its error word stays clear.  Collected last on
purpose, and written to pass both alone in a fresh process and after every other test."""
import ctypes

import numpy as np
import pytest
import torch

import oracle
from helpers import check_gemm_tolerance, make_packed, make_x, to_dev

pytestmark = pytest.mark.gpu


def _call_static(lib, x, qw, zs, bias, out, M, N, K, g):
    return lib.w4a16_gemm_static_scratch(x.data_ptr(), qw.data_ptr(), zs.data_ptr(),
                                         None if bias is None else bias.data_ptr(), out.data_ptr(), M, N, K, g,
                                         torch.cuda.current_stream().cuda_stream)


def test_static_scratch_entry_point_matches_regular_entry_point():
    import quant
    lib = quant.load_library()
    g = 128
    cases = [(300, 384, 2048), (200, 1024, 4096)]          # (tokens, N, K): two different problems, back to back
    for round_ in range(2):                                   # and the whole sequence twice: stale scratch contents
        for M, N, K in cases:
            p = make_packed(N, K, g, seed=900 + N)
            qw, zs = to_dev(p)
            x = make_x(M, K, seed=77 + round_).cuda()[0].contiguous()
            bias = (torch.randn(N, generator=torch.Generator().manual_seed(3)) * 0.02).half().cuda()
            ref = torch.empty(M, N, dtype=torch.float16, device="cuda")
            st = lib.w4a16_gemm_algo(x.data_ptr(), qw.data_ptr(), zs.data_ptr(), bias.data_ptr(), ref.data_ptr(),
                                     M, N, K, g, None, 0, torch.cuda.current_stream().cuda_stream, 2)
            assert st == 0
            out = torch.full((M + 2, N), 555.0, dtype=torch.float16, device="cuda")
            assert _call_static(lib, x, qw, zs, bias, out[1:M + 1], M, N, K, g) == 0
            torch.cuda.synchronize()
            assert (out[0] == 555.0).all() and (out[M + 1] == 555.0).all()         # nothing written outside
            # same tolerance as every GEMM parity test (the K split only re-associates the fp32 sum): against the
            # regular entry point and against the oracle's dequantise-then-matmul
            check_gemm_tolerance(out[1:M + 1], ref, x, p["w_deq"], K)
            want = oracle.gemm_f16(x.cpu().unsqueeze(0), p["w_deq"], bias.cpu().unsqueeze(0)).astype(np.float32)
            check_gemm_tolerance(out[1:M + 1], want, x, p["w_deq"], K)
            again = torch.empty(M, N, dtype=torch.float16, device="cuda")
            assert _call_static(lib, x, qw, zs, bias, again, M, N, K, g) == 0
            torch.cuda.synchronize()
            assert torch.equal(again, out[1:M + 1])                                 # second call in a row: identical
    flag = ctypes.c_int(-1)
    assert lib.w4a16_static_scratch_error_flag(ctypes.byref(flag)) == 0 and flag.value == 0


def test_static_scratch_entry_point_rejects_what_does_not_fit():
    import quant
    lib = quant.load_library()
    t = torch.zeros(4096, dtype=torch.float16, device="cuda")
    p = t.data_ptr()
    sp = torch.cuda.current_stream().cuda_stream
    # 2 * 4096 * 4096 * 4 B = 128 MiB of partial tiles > 16 MiB
    assert lib.w4a16_gemm_static_scratch(p, p, p, None, p, 4096, 4096, 4096, 128, sp) == 9
    assert lib.w4a16_status_str(9) == b"size exceeds a fixed capacity of this entry point"
    assert lib.w4a16_gemm_static_scratch(p, p, p, None, p, 64, 256, 512, 128, sp) == 2      # K too short to split
    assert lib.w4a16_gemm_static_scratch(p, p, p, None, p, 64, 256, 2048, 32, sp) == 3      # group size
    assert lib.w4a16_gemm_static_scratch(None, p, p, None, p, 64, 256, 2048, 128, sp) == 1
