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
