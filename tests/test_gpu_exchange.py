"""The decode GEMV fused with its all-reduce, and the exchange all-gather, on ONE GPU: a single-rank exchange
runs the whole protocol (push, flag, wait, ordered sum, epoch flip) against this GPU's own buffer.  With one
rank the sum has one term, so the output must equal the plain decode kernel's bit for bit.  The multi-rank
behaviour is covered by test_gpu_tp_exchange.py (needs two GPUs) and the host logic by the CPU gloo tests."""
import ctypes

import pytest
import torch

from helpers import make_packed, make_x, to_dev

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def exchange():
    from w4a16.tp import PeerExchange
    ex = PeerExchange(32 * 4096)
    yield ex
    ex.close()


CASES = [(1, 4096, 4096, 128, 4096), (8, 1024, 2048, 64, 2048), (16, 512, 16384, 128, 16384), (32, 256, 1344, 64, 1408),
         (5, 4096, 512, 128, 512)]


def test_single_rank_exchange_equals_plain_kernel(exchange):
    import quant
    calls0, err = exchange.status()
    assert err == 0
    n_calls = 0
    for rep in range(2):
        for M, N, K, g, k_config in CASES:
            p = make_packed(N, K, g, seed=40 + N % 7)
            qw, zs = to_dev(p)
            x = make_x(M, K, seed=rep).cuda()
            bias = (torch.randn(1, N, generator=torch.Generator().manual_seed(2)) * 0.05).half().cuda()
            ref = quant.gemm_awq_bias(x, qw, zs, bias, N, g, algo=quant.ALGO_SKINNY)
            out = quant.gemm_awq_allreduce(x, qw, zs, bias, N, g, k_config, exchange.buffers, 1, 0, exchange.capacity)
            n_calls += 1
            if k_config == K:
                assert torch.equal(out, ref), (M, N, K)
            else:       # launch shape chosen for a larger K: another split of the same sum
                assert torch.allclose(out.float(), ref.float(), atol=2e-2, rtol=2e-2)
    torch.cuda.synchronize()
    calls1, err = exchange.status()
    assert err == 0 and calls1 - calls0 == n_calls            # one epoch per call: both buffer halves were used


def test_exchange_calls_replay_in_a_cuda_graph(exchange):
    import quant
    M, N, K, g = 8, 2048, 4096, 128
    p = make_packed(N, K, g, seed=3)
    qw, zs = to_dev(p)
    x = make_x(M, K).cuda()
    ref = quant.gemm_awq_bias(x, qw, zs, None, N, g, algo=quant.ALGO_SKINNY)
    outs = [torch.zeros(1, M, N, dtype=torch.float16, device="cuda") for _ in range(3)]
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        gathered = exchange.allgather(torch.arange(16, device="cuda", dtype=torch.float32))
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for o in outs:                                     # odd number of calls: successive replays start on
                quant.gemm_awq_allreduce(x, qw, zs, None, N, g, K, exchange.buffers, 1, 0, exchange.capacity, out=o,
                                         static_weights=True)  # alternating buffer halves
        for _ in range(3):
            for o in outs:
                o.zero_()
            graph.replay()
            side.synchronize()
            for o in outs:
                assert torch.equal(o, ref)
    torch.cuda.current_stream().wait_stream(side)
    assert torch.equal(gathered, torch.arange(16, device="cuda", dtype=torch.float32)[None])
    assert exchange.status()[1] == 0


def test_exchange_argument_errors(exchange):
    import quant
    lib = quant.load_library()
    p = make_packed(256, 512, 128, seed=1)
    qw, zs = to_dev(p)
    with pytest.raises(RuntimeError):
        quant.gemm_awq_allreduce(make_x(33, 512).cuda(), qw, zs, None, 256, 128, 512, exchange.buffers, 1, 0, exchange.capacity)
    x = make_x(8, 512).cuda()
    out = torch.empty(8, 256, dtype=torch.float16, device="cuda")
    sp = torch.cuda.current_stream().cuda_stream
    args = (x.data_ptr(), qw.data_ptr(), zs.data_ptr(), None, out.data_ptr(), 8, 256, 512, 128)
    assert lib.w4a16_gemm_allreduce(*args, 512, exchange.buffers, 1, 0, 8 * 256 - 1, sp, 0) == 9      # capacity too small
    assert lib.w4a16_gemm_allreduce(*args, 256, exchange.buffers, 1, 0, exchange.capacity, sp, 0) == 2  # k_config < K
    assert lib.w4a16_gemm_allreduce(*args, 512, exchange.buffers, 9, 0, exchange.capacity, sp, 0) == 2  # world > 8
    assert lib.w4a16_gemm_allreduce(*args, 512, exchange.buffers, 2, 0, exchange.capacity, sp, 0) == 1  # rank 1's buffer missing
    assert lib.w4a16_exchange_bytes(9, 10) == 0
    buf = ctypes.c_void_p()
    assert lib.w4a16_exchange_alloc(2, 0, ctypes.byref(buf)) == 2


def test_allreduce_supported_predicate():
    """The host-side predicate agrees with what the fused call accepts: decode-sized shards yes, more than 32 tokens
    or a shard whose grid cannot be resident in one wave no."""
    import quant
    lib = quant.load_library()
    assert lib.w4a16_allreduce_supported(8, 4096, 2048, 2048, 128, 8) == 1
    assert lib.w4a16_allreduce_supported(32, 4096, 1344, 1408, 64, 8) == 1      # the short shard of 11008 @ g=64 over 8 ranks
    assert lib.w4a16_allreduce_supported(33, 4096, 2048, 2048, 128, 8) == 0
    assert lib.w4a16_allreduce_supported(8, 4096, 2048, 1024, 128, 8) == 0      # k_config below K
    assert lib.w4a16_allreduce_supported(8, 4096, 2048, 2048, 128, 9) == 0      # more ranks than the buffers hold
