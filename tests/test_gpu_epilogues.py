"""The fused epilogues of w4a16_gemm_fused (residual add, SwiGLU product) against the oracle, through the Python shim
(i.e. the C ABI).  The reference carries both as hooks around its kernel (gemm_awq_residual_ut, gemm_awq_silu_dot_ut in
quantization/nvidia/script/gemm_awq_test.py:53-72) and checks them against torch with allclose(2e-2, 2e-2)."""
import numpy as np
import pytest
import torch

import oracle
from helpers import check_gemm_tolerance, make_packed, make_x, to_dev

pytestmark = pytest.mark.gpu


def _lin(p, bias=None):
    from w4a16.tp import _from_buffers
    qw, zs = to_dev(p)
    return _from_buffers(qw, zs, bias, p["g"])


@pytest.mark.parametrize("M,algo", [(1, 1), (7, 1), (8, 1), (16, 1), (32, 1), (100, 2), (300, 2)])
@pytest.mark.parametrize("N,K,g", [(256, 512, 128), (1376, 1408, 64)])
def test_residual_epilogue(M, algo, N, K, g):
    """out = (fp16(acc) + bias) + residual with both adds in fp16, in every kernel."""
    import quant
    p = make_packed(N, K, g, seed=61 + N)
    qw, zs = to_dev(p)
    x = make_x(M, K, seed=5)
    gen = torch.Generator().manual_seed(9)
    b = (torch.randn(1, N, generator=gen) * 0.02).half()
    r = torch.randn(1, M, N, generator=gen).half()
    out = quant.gemm_awq_bias(x.cuda(), qw, zs, b.cuda(), N, g, algo=algo, residual=r.cuda())
    plain = quant.gemm_awq_bias(x.cuda(), qw, zs, b.cuda(), N, g, algo=algo)
    torch.cuda.synchronize()
    assert torch.equal(out, plain + r.cuda())                       # exactly the separate fp16 add it replaces
    ref = oracle.gemm_f16(x, p["w_deq"], b).astype(np.float32) + r[0].float().numpy()
    err = np.abs(out[0].float().cpu().numpy() - ref).max()
    assert err <= 2e-2 + 1e-2 * float(x.abs().max()) * (K ** 0.5) * float(np.abs(p["w_deq"].astype(np.float32)).max())


@pytest.mark.parametrize("kernel", [1, 2])                          # both decode kernels
@pytest.mark.parametrize("M", [1, 5, 8, 16, 32])
@pytest.mark.parametrize("n,K,g,bias", [(128, 512, 128, False), (704, 1024, 64, True), (2752, 4096, 64, False)])
def test_swiglu_epilogue(kernel, M, n, K, g, bias):
    """A fuse_gate_up linear with W4A16_FLAG_SILU_MUL returns fp16(silu(gate)) * up: bit-equal to the plain GEMV
    followed by the SwiGLU product kernel on the de-interleaved output, and within tolerance of the oracle."""
    import quant
    from w4a16.tp import fuse_gate_up, split_gate_up
    pg, pu = make_packed(n, K, g, seed=70 + n), make_packed(n, K, g, seed=71 + n)
    gen = torch.Generator().manual_seed(4)
    bg = (torch.randn(1, n, generator=gen) * 0.02).half().cuda() if bias else None
    bu = (torch.randn(1, n, generator=gen) * 0.02).half().cuda() if bias else None
    fused = fuse_gate_up(_lin(pg, bg), _lin(pu, bu))
    x = (make_x(M, K, seed=8) * 0.5).cuda()
    lib = quant.load_library()
    try:
        lib.w4a16_tune_decode(kernel, 0, 0, 0)
        got = fused(x, silu_mul=True)
        plain = fused(x)
    finally:
        lib.w4a16_tune_decode(0, 0, 0, 0)
    torch.cuda.synchronize()
    assert tuple(got.shape) == (1, M, n)
    gate, up = split_gate_up(plain)
    assert torch.equal(got, quant.silu_mul(torch.cat((gate, up), dim=-1).contiguous()))
    og = oracle.gemm_f16(x.cpu(), pg["w_deq"], None if bg is None else bg.cpu()).astype(np.float32)
    ou = oracle.gemm_f16(x.cpu(), pu["w_deq"], None if bu is None else bu.cpu()).astype(np.float32)
    ref = og / (1.0 + np.exp(-og)) * ou
    assert np.allclose(got[0].float().cpu().numpy(), ref, atol=2e-2, rtol=2e-2)


def test_swiglu_epilogue_rejects_what_it_cannot_do():
    import quant
    p = make_packed(128, 256, 64, seed=3)
    qw, zs = to_dev(p)
    x = make_x(40, 256).cuda()
    with pytest.raises(RuntimeError):
        quant.gemm_awq_bias(x, qw, zs, None, 128, 64, silu_mul=True)                       # 40 tokens: not a decode pass
    p96 = make_packed(96, 256, 64, seed=3)
    qw96, zs96 = to_dev(p96)
    with pytest.raises(RuntimeError):
        quant.gemm_awq_bias(x[:, :4].contiguous(), qw96, zs96, None, 96, 64, silu_mul=True)  # odd number of tiles


@pytest.mark.parametrize("rms", [False, True])
@pytest.mark.parametrize("M,H,N,K0,g", [(1, 512, 256, 256, 128), (5, 4096, 512, 1024, 128), (8, 4096, 1376, 2048, 64),
                                        (16, 4096, 256, 4096, 128), (8, 8192, 256, 512, 128), (3, 5120, 512, 640, 64)])
def test_residual_stats_then_prenorm_gemv(rms, M, H, N, K0, g):
    """Producer GEMV (K0 -> H, residual add, row statistics out) followed by the consumer GEMV that normalises its
    input from those statistics (H -> N): against the launches they replace (GEMV, add, add_norm, GEMV) and against
    the oracle on a float64 normalisation."""
    import quant
    p0, p1 = make_packed(H, K0, g, seed=31 + H + K0), make_packed(N, H, g, seed=32 + N + H)
    qw0, zs0 = to_dev(p0)
    qw1, zs1 = to_dev(p1)
    gen = torch.Generator().manual_seed(12 + M)
    x0 = make_x(M, K0, seed=3 + M).cuda()
    res = (torch.randn(1, M, H, generator=gen) * 1.3 + 0.2).half().cuda()
    w = (1.0 + 0.1 * torch.randn(H, generator=gen)).half()
    b = None if rms else (0.05 * torch.randn(H, generator=gen)).half()
    bias = (torch.randn(1, N, generator=gen) * 0.02).half().cuda()
    eps = 1e-6 if rms else 1e-5
    stats = quant.row_stats_buffer(H, "cuda")
    launches0 = quant.launch_count()
    h = quant.gemm_awq_bias(x0, qw0, zs0, None, H, g, residual=res, stats_out=stats)
    got = quant.gemm_awq_bias(h, qw1, zs1, bias, N, g, relu=True, pre_norm=(w.cuda(), None if b is None else b.cuda(), eps, rms, stats))
    assert quant.launch_count() - launches0 == 2                    # two launches, not three
    lib = quant.load_library()
    try:
        lib.w4a16_tune_decode(1, 0, 0, 0)                           # the kernel that writes statistics, without them
        h_plain = quant.gemm_awq_bias(x0, qw0, zs0, None, H, g, residual=res)
    finally:
        lib.w4a16_tune_decode(0, 0, 0, 0)
    assert torch.equal(h, h_plain)                                  # the statistics do not change the output
    # the statistics themselves: per row sum and sum of squares of h, added over the parts
    torch.cuda.synchronize()
    parts = int(stats[:1].view(torch.int32).item())
    data = stats[4:4 + parts * 32].view(parts, 16, 2).double().sum(0)[:M].cpu()
    hd = h[0].double().cpu()
    assert torch.allclose(data[:, 0], hd.sum(-1), rtol=1e-5, atol=1e-2)
    assert torch.allclose(data[:, 1], (hd * hd).sum(-1), rtol=1e-5, atol=1e-2)
    hn_two = quant.add_norm(h, None, w.cuda(), None if b is None else b.cuda(), eps, rms)[1]
    two = quant.gemm_awq_bias(hn_two, qw1, zs1, bias, N, g, relu=True)
    torch.cuda.synchronize()
    # one-pass variance and a different summation order: the normalised inputs may differ in the last fp16 bit of a
    # few elements, the outputs by far less than the GEMM tolerance
    scale = float(np.abs(p1["w_deq"].astype(np.float32)).max()) * (H ** 0.5) * 4.0
    assert float((got.float() - two.float()).abs().max()) <= 2e-3 * scale + 1e-3
    x64 = hd
    if rms:
        hn = (w.double() * (x64 * torch.rsqrt((x64 * x64).mean(-1, keepdim=True) + eps)).half().double()).half()
    else:
        mu = x64.mean(-1, keepdim=True)
        var = ((x64 - mu) ** 2).mean(-1, keepdim=True)
        hn = ((x64 - mu) * torch.rsqrt(var + eps) * w.double() + b.double()).half()
    ref = np.maximum(oracle.gemm_f16(hn.unsqueeze(0), p1["w_deq"], bias.cpu()).astype(np.float32), 0.0)
    check_gemm_tolerance(got[0].float().cpu().numpy(), ref, hn.unsqueeze(0), p1["w_deq"], H)


def test_prenorm_falls_back_beyond_sixteen_tokens():
    """More tokens than one pass of the decode kernel: the shim runs the normalisation as its own launch, and the
    C entry points refuse."""
    import quant
    N, K, g, M = 256, 4096, 128, 17
    p = make_packed(N, K, g, seed=3)
    qw, zs = to_dev(p)
    gen = torch.Generator().manual_seed(2)
    x = torch.randn(1, M, K, generator=gen).half().cuda()
    w = (1.0 + 0.1 * torch.randn(K, generator=gen)).half().cuda()
    stats = quant.row_stats_buffer(K, "cuda")
    assert not quant.prenorm_supported(M, K)
    got = quant.gemm_awq_bias(x, qw, zs, None, N, g, pre_norm=(w, None, 1e-6, True, stats))
    two = quant.gemm_awq_bias(quant.add_norm(x, None, w, None, 1e-6, True)[1], qw, zs, None, N, g)
    assert torch.equal(got, two)
    lib = quant.load_library()
    out = torch.empty(1, M, N, dtype=torch.float16, device="cuda")
    st = lib.w4a16_gemm_prenorm(x.data_ptr(), stats.data_ptr(), w.data_ptr(), None, 1e-6, 1, qw.data_ptr(), zs.data_ptr(), None,
                                out.data_ptr(), M, N, K, g, None, 0)
    assert st == 6                                                  # W4A16_ERR_BAD_ALGO
    st = lib.w4a16_gemm_residual_stats(x.data_ptr(), qw.data_ptr(), zs.data_ptr(), None, None, out.data_ptr(), stats.data_ptr(),
                                       M, N, K, g, None, 0)
    assert st == 6


@pytest.mark.parametrize("M", [1, 6, 8, 16, 32])
def test_row_parallel_residual_single_rank_exchange(M):
    """The residual add inside the GEMV fused with its all-reduce (one rank: the exchange path on one GPU)."""
    import quant
    from w4a16.tp import PeerExchange
    N, K, g = 512, 1024, 128
    p = make_packed(N, K, g, seed=77)
    qw, zs = to_dev(p)
    gen = torch.Generator().manual_seed(5)
    x = make_x(M, K, seed=6).cuda()
    r = torch.randn(1, M, N, generator=gen).half().cuda()
    ex = PeerExchange(32 * N)
    stats = quant.row_stats_buffer(N, "cuda") if M <= 16 else None
    got = quant.gemm_awq_allreduce(x, qw, zs, None, N, g, K, ex.buffers, 1, 0, ex.capacity, residual=r, stats_out=stats)
    lib = quant.load_library()
    try:
        if stats is not None:
            lib.w4a16_tune_decode(1, 0, 0, 0)                       # the kernel that writes statistics, without them
        plain = quant.gemm_awq_allreduce(x, qw, zs, None, N, g, K, ex.buffers, 1, 0, ex.capacity)
    finally:
        lib.w4a16_tune_decode(0, 0, 0, 0)
    torch.cuda.synchronize()
    assert torch.equal(got, plain + r)
    if stats is not None:
        parts = int(stats[:1].view(torch.int32).item())
        data = stats[4:4 + parts * 32].view(parts, 16, 2).double().sum(0)[:M].cpu()
        assert torch.allclose(data[:, 0], got[0].double().sum(-1).cpu(), rtol=1e-5, atol=1e-2)
