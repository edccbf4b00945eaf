"""Decode attention kernel against the float64 definition (oracle.decode_attention): scores, softmax, weighted sum,
the append of the new key/value row to the static cache, rotary embedding, and the fused-qkv input layout.

Tolerance (floating point, stated): |out - ref| <= 2e-3 * max|v| + 2^-10 * |ref|  - one fp16 rounding of the output
plus the fp16 rounding of the rotated key stored in the cache; cache rows must equal the oracle's fp16 rows exactly
where no rotary embedding is applied, and within one fp16 ulp with it (fp32 vs float64 rotation)."""
import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu


def _case(B, H, D, L, pos, rope, seed, pad=0):
    import quant
    g = torch.Generator().manual_seed(seed)
    qkv = torch.randn(B, 3 * H * D + pad, generator=g).half()
    kc = torch.randn(B, H, L, D, generator=g).half()
    vc = torch.randn(B, H, L, D, generator=g).half()
    cos = sin = None
    if rope:
        ang = torch.rand(L, D // 2, generator=g) * 6.28
        emb = torch.cat((ang, ang), dim=-1)
        cos, sin = emb.cos().half(), emb.sin().half()
    q, k, v = (qkv[:, i * H * D:(i + 1) * H * D].reshape(B, H, D).numpy() for i in range(3))
    ref, k_row, v_row = oracle.decode_attention(q, k, v, kc.numpy(), vc.numpy(), pos, D ** -0.5,
                                                None if cos is None else cos[pos].numpy(), None if sin is None else sin[pos].numpy())
    kd, vd = kc.cuda(), vc.cuda()
    out = quant.decode_attention(qkv.cuda(), kd, vd, torch.tensor([pos], device="cuda"), H,
                                 rope=None if cos is None else (cos.cuda(), sin.cuda()))
    torch.cuda.synchronize()
    got = out.float().cpu().numpy().reshape(B, H, D)
    tol = 2e-3 * float(np.abs(vc.numpy()[:, :, :pos + 1]).max()) + 2.0 ** -10 * np.abs(ref)
    assert (np.abs(got - ref) <= tol).all(), float(np.abs(got - ref).max())
    # the cache: row `pos` appended, every other row untouched
    kn, vn = kd.cpu().numpy(), vd.cpu().numpy()
    assert np.array_equal(vn[:, :, pos], v_row)
    if rope:
        assert np.allclose(kn[:, :, pos].astype(np.float32), k_row.astype(np.float32), rtol=2e-3, atol=2e-3)
    else:
        assert np.array_equal(kn[:, :, pos], k_row)
    mask = np.ones(L, dtype=bool)
    mask[pos] = False
    assert np.array_equal(kn[:, :, mask], kc.numpy()[:, :, mask]) and np.array_equal(vn[:, :, mask], vc.numpy()[:, :, mask])


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("rope", [False, True])
def test_decode_attention_matches_definition(D, rope):
    for pos in (0, 1, 31, 32, 255, 300, 639):
        _case(B=3, H=4, D=D, L=640, pos=pos, rope=rope, seed=pos + D)


def test_decode_attention_long_cache_and_padded_rows():
    _case(B=2, H=2, D=128, L=4096, pos=4095, rope=True, seed=1)
    _case(B=1, H=32, D=128, L=1280, pos=1279, rope=False, seed=2, pad=64)     # qkv row stride larger than 3*H*D


def test_decode_attention_argument_errors():
    import quant
    lib = quant.load_library()
    t = torch.zeros(3 * 4 * 128 * 2, dtype=torch.float16, device="cuda")
    pos = torch.zeros(1, dtype=torch.int64, device="cuda")
    p, sp = t.data_ptr(), torch.cuda.current_stream().cuda_stream
    call = lib.w4a16_decode_attention
    assert call(p, p, p, p, pos.data_ptr(), None, None, 1, 4, 96, 8, 3 * 4 * 96, 0.1, sp) == 2       # head_dim
    assert call(p, p, p, p, pos.data_ptr(), None, None, 1, 4, 128, 8, 3 * 4 * 128 - 1, 0.1, sp) == 2  # row stride too short
    assert call(p, p, p, p, None, None, None, 1, 4, 128, 8, 3 * 4 * 128, 0.1, sp) == 1
    assert call(p, p, p, p, pos.data_ptr(), p, None, 1, 4, 128, 8, 3 * 4 * 128, 0.1, sp) == 1         # cos without sin
    assert call(p, p, p, p, pos.data_ptr(), None, None, 1, 4, 128, 60000, 3 * 4 * 128, 0.1, sp) == 9   # scores do not fit
    with pytest.raises(RuntimeError):
        quant.decode_attention(t.view(2, -1), torch.zeros(2, 4, 8, 128, dtype=torch.float16, device="cuda"),
                               torch.zeros(2, 4, 8, 128, dtype=torch.float16, device="cuda"), pos.int(), 4)


@pytest.mark.parametrize("rms", [False, True])
@pytest.mark.parametrize("rows,cols", [(8, 4096), (32, 4096), (3, 512), (1, 8192), (5, 264)])
def test_add_norm_matches_torch(rms, rows, cols):
    """Residual add + LayerNorm / RMSNorm in one launch against the torch ops it replaces.  Tolerance: the sum must be
    bit-equal (one fp16 add); the normalised output within 2 fp16 ulps of torch's (fp32 statistics, different
    summation order)."""
    import quant
    g = torch.Generator().manual_seed(rows + cols)
    x = torch.randn(rows, cols, generator=g).half().cuda()
    d = (torch.randn(rows, cols, generator=g) * 0.5).half().cuda()
    w = (1 + 0.1 * torch.randn(cols, generator=g)).half().cuda()
    b = (0.1 * torch.randn(cols, generator=g)).half().cuda()
    for delta in (d, None):
        s_ref = x + delta if delta is not None else x
        if rms:
            v = s_ref.float()
            h_ref = w * (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + 1e-6)).half()
        else:
            h_ref = torch.nn.functional.layer_norm(s_ref, (cols,), w, b, 1e-5)
        s, h = quant.add_norm(x, delta, w, b, 1e-6 if rms else 1e-5, rms)
        assert torch.equal(s, s_ref)
        err = (h.float() - h_ref.float()).abs()
        assert (err <= 2.0 ** -9 * h_ref.float().abs() + 1e-3).all(), err.max().item()
    lib = quant.load_library()
    sp = torch.cuda.current_stream().cuda_stream
    assert lib.w4a16_add_norm(x.data_ptr(), None, None, x.data_ptr(), w.data_ptr(), None, 1, 8200, 1e-5, 0, sp) == 9
    assert lib.w4a16_add_norm(x.data_ptr(), None, None, x.data_ptr(), w.data_ptr(), None, 1, 100, 1e-5, 0, sp) == 2
    assert lib.w4a16_add_norm(x.data_ptr(), d.data_ptr(), None, x.data_ptr(), w.data_ptr(), None, 1, 64, 1e-5, 0, sp) == 1


def test_silu_mul_and_relu_epilogue():
    import quant
    from helpers import make_packed, make_x, to_dev
    g = torch.Generator().manual_seed(3)
    gu = torch.randn(5, 2 * 1376, generator=g).half().cuda()
    ref = torch.nn.functional.silu(gu[:, :1376]) * gu[:, 1376:]
    got = quant.silu_mul(gu)
    assert (got.float() - ref.float()).abs().max().item() <= 2e-3 and got.shape == (5, 1376)
    # ReLU fused into the GEMM epilogue: exactly max(plain output, 0), both kernels
    for M, algo in ((8, quant.ALGO_SKINNY), (96, quant.ALGO_TC)):
        p = make_packed(512, 1024, 128, seed=9)
        qw, zs = to_dev(p)
        x = make_x(M, 1024).cuda()
        bias = (torch.randn(1, 512, generator=g) * 0.05).half().cuda()
        plain = quant.gemm_awq_bias(x, qw, zs, bias, 512, 128, algo=algo)
        fused = quant.gemm_awq_bias(x, qw, zs, bias, 512, 128, algo=algo, relu=True)
        assert torch.equal(fused, torch.relu(plain)) and (plain < 0).any()


def test_decode_attention_context_split_over_a_cluster():
    """The positions of one (head, sequence) split over 2/4/8 CTAs of a cluster and recombined: same tolerance as
    the single-CTA form, including positions smaller than the split (ranks with nothing to do)."""
    import quant
    lib = quant.load_library()
    try:
        for split in (1, 2, 4, 8):
            lib.w4a16_tune_attention(split)
            for pos in (0, 2, 5, 63, 64, 500, 639):
                _case(B=2, H=3, D=128, L=640, pos=pos, rope=(pos % 2 == 0), seed=pos + split)
            _case(B=2, H=3, D=64, L=320, pos=319, rope=True, seed=split)
    finally:
        lib.w4a16_tune_attention(0)
