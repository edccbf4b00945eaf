"""GPU packers and the standalone dequantiser against the CPU oracle: byte-identical."""
import numpy as np
import pytest
import torch

import oracle
from helpers import make_packed, make_weight, to_dev

pytestmark = pytest.mark.gpu

SHAPES = [(64, 128, 128), (96, 256, 64), (32, 32, 32), (4096, 1024, 128), (1376, 1408, 64), (4096, 4096, 128)]


@pytest.mark.parametrize("N,K,g", SHAPES)
def test_pack_flow_matches_oracle(N, K, g):
    import quant
    from w4a16 import quant_lmdeploy
    w = make_weight(N, K, seed=N + K)
    qw8, zeros, scales, w_fp16 = oracle.generate_quant(w, 4, g)
    o_zs = oracle.transpose_merge_zeros_scales(zeros, scales, K, N, g)
    o_awq = oracle.convert_ours_to_awq(qw8, K, N)
    o_lmd = oracle.convert_awq_to_lmdeploy(o_awq, K, N) if N * K <= 4096 * 1024 else None

    d_zs = torch.empty((K // g, 2 * N), dtype=torch.float16, device="cuda")
    quant.transpose_merge_zeros_scales(zeros.cuda(), scales.cuda(), d_zs, K, N, g)
    assert np.array_equal(d_zs.cpu().numpy().view(np.uint16), o_zs)
    d_awq = torch.empty((K, N // 2), dtype=torch.uint8, device="cuda")
    quant.convert_ours_to_awq(qw8.cuda(), d_awq, K, N)
    assert np.array_equal(d_awq.cpu().numpy().view(np.uint32), o_awq)
    d_lmd = torch.empty((K, N // 8), dtype=torch.int32, device="cuda")
    quant.convert_awq_to_lmdeploy(d_awq, d_lmd, K, N)
    if o_lmd is not None:
        assert np.array_equal(d_lmd.cpu().numpy().view(np.uint32), o_lmd)
    # whatever the size: unpacking the GPU result through the closed form gives the quantizer's q
    q = oracle.unpack(d_lmd.cpu().numpy(), K, N)
    expect = np.empty((N, K), dtype=np.uint8)
    expect[:, 0::2] = qw8.numpy() >> 4
    expect[:, 1::2] = qw8.numpy() & 0xF
    assert np.array_equal(q, expect)

    # the module-level flows give the same tensors: the reference's step sequence (torch fp16 quantizer on the GPU +
    # the three layout kernels) and the single fused quantise-and-pack kernel
    for fused in (False, True):
        m_qw, m_zs, m_wfp16 = quant_lmdeploy(w.cuda(), K, N, g, 4, fused=fused)
        assert np.array_equal(m_qw.cpu().numpy(), d_lmd.cpu().numpy()), fused
        assert np.array_equal(m_zs.cpu().numpy().view(np.uint16), o_zs), fused
        assert torch.equal(m_wfp16.cpu(), w_fp16), fused
    # and the fused kernel's optional outputs are generate_quant's tensors
    _, _, _, f_ours, f_zeros, f_scales = quant.quantize_pack(w.cuda(), K, N, g, parts=True)
    assert torch.equal(f_ours.cpu(), qw8) and torch.equal(f_zeros.cpu(), zeros) and torch.equal(f_scales.cpu(), scales)


def test_fused_quantize_pack_matches_reference_golden_vectors():
    """The single-kernel quantise-and-pack against the vectors made by the reference itself: its Python quantizer
    (golden_quantizer.npz) and its own CUDA layout kernels run on a B200 (golden_reference_cuda.npz), on all golden
    cases including the crafted one whose scales are denormal."""
    import os
    import quant
    from golden.make_golden import QUANT_CASES, seeded_weight
    here = os.path.dirname(os.path.abspath(__file__))
    gold_q = np.load(os.path.join(here, "golden", "golden_quantizer.npz"))
    gold_c = np.load(os.path.join(here, "golden", "golden_reference_cuda.npz"))
    for i, (N, K, g, seed, std) in enumerate(QUANT_CASES):
        w = seeded_weight(N, K, seed, std).cuda()
        qw, zs, w_fp16, ours, zeros, scales = quant.quantize_pack(w, K, N, g, parts=True)
        assert np.array_equal(ours.cpu().numpy(), gold_q[f"c{i}_qweight"]), i
        assert np.array_equal(zeros.cpu().numpy().view(np.uint16), gold_q[f"c{i}_zeros"]), i
        assert np.array_equal(scales.cpu().numpy().view(np.uint16), gold_q[f"c{i}_scales"]), i
        assert np.array_equal(w_fp16.cpu().numpy().view(np.uint16), gold_q[f"c{i}_wfp16"]), i
        assert np.array_equal(zs.cpu().numpy().view(np.uint16), gold_c[f"c{i}_zs"]), i
        assert np.array_equal(qw.cpu().numpy(), gold_c[f"c{i}_lmdeploy"]), i


def test_fused_quantize_pack_degenerate_groups():
    """Constant groups (max == min: the 1e-5 clamp and an infinite min / scale), all-zero groups, groups that are
    all negative or all positive, fp16 extremes: bit-identical to the reference's statement of the quantizer."""
    import quant
    N, K, g = 64, 256, 64
    gen = torch.Generator().manual_seed(11)
    w = (torch.randn(N, K, generator=gen) * 0.02).half()
    w[0] = 0.5; w[1] = -0.5; w[2] = 0.0; w[3, :64] = 1e-4; w[4] = w[4].abs() + 1.0; w[5] = -w[5].abs() - 1.0
    w[6, 0] = 60000.0; w[7, 1] = -60000.0; w[8, :128] = 6e-8; w[9] = torch.linspace(-1, 1, K).half()
    qw8, zeros, scales, w_fp16 = oracle.generate_quant(w, 4, g)
    o_qw, o_zs = oracle.pack(qw8, zeros, scales, K, N, g)
    qw, zs, d_wfp16, ours, d_zeros, d_scales = quant.quantize_pack(w.cuda(), K, N, g, parts=True)
    assert torch.equal(ours.cpu(), qw8)
    # zero points compare as numbers: torch's clamp of -round(x) may hand back -0.0 where x rounds to zero, the kernel
    # always writes +0.0 (the packed value zero + 64 is the same either way, checked below)
    assert np.array_equal(d_zeros.cpu().numpy().astype(np.float32), zeros.numpy().astype(np.float32))
    assert np.array_equal(d_scales.cpu().numpy().view(np.uint16), scales.numpy().view(np.uint16))
    assert np.array_equal(d_wfp16.cpu().numpy().view(np.uint16), w_fp16.numpy().view(np.uint16))
    assert np.array_equal(qw.cpu().numpy().view(np.uint32), o_qw) and np.array_equal(zs.cpu().numpy().view(np.uint16), o_zs)


@pytest.mark.parametrize("N,K,g", SHAPES)
def test_dequant_bit_exact(N, K, g):
    import quant
    p = make_packed(N, K, g, seed=7 + N)
    qw, zs = to_dev(p)
    w = quant.dequant(qw, zs, N, K, g)
    assert np.array_equal(w.cpu().numpy().view(np.uint16), p["w_deq"].view(np.uint16))
    # and equals the quantizer's own dequantised weight (no denormal scales in this data)
    assert np.array_equal(w.cpu().numpy().view(np.uint16), p["w_fp16"].numpy().view(np.uint16))


def test_dequant_crafted_edge_cases():
    """All 16 nibble values x zero points {0, 7, 15}; denormal / tiny / huge scales (FTZ regime);
    non-integer zero points (exercise the fp16 rounding of the subtraction)."""
    import quant
    N, K, g = 32, 128, 32
    rng = np.random.default_rng(3)
    q = np.tile(np.arange(16, dtype=np.uint8), (N, K // 16))
    qw8 = torch.from_numpy(((q[:, 0::2] << 4) | q[:, 1::2]).astype(np.uint8))
    zero_vals = np.array([0, 7, 15, 3.5, 0.0625, 14.9375], dtype=np.float16)
    scale_bits = np.array([0x0001, 0x03FF, 0x0400, 0x0401, 0x1400, 0x2E66, 0x3C00, 0x7BFF, 0x5000, 0x8001, 0xBC00],
                          dtype=np.uint16)
    zeros = torch.from_numpy(zero_vals[rng.integers(0, len(zero_vals), (N, K // g))])
    scales = torch.from_numpy(scale_bits[rng.integers(0, len(scale_bits), (N, K // g))].view(np.float16))
    qweight, zs = oracle.pack(qw8, zeros, scales, K, N, g)
    expect = oracle.dequant(qweight, zs, K, N, g)
    got = quant.dequant(torch.from_numpy(qweight.view(np.int32)).cuda(),
                        torch.from_numpy(zs.view(np.float16)).cuda(), N, K, g)
    assert np.array_equal(got.cpu().numpy().view(np.uint16), expect.view(np.uint16))
