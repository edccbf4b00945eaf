"""Pins the CPU oracle: against vectors produced by the reference's own Python quantizer
(golden_quantizer.npz) and by the reference's own CUDA extension run on a B200
(golden_reference_cuda.npz, present once generated on a GPU box)."""
import os

import numpy as np
import pytest
import torch

import oracle
from golden.make_golden import QUANT_CASES, GEMM_TOKENS, seeded_weight, seeded_x
from helpers import check_gemm_tolerance

HERE = os.path.dirname(os.path.abspath(__file__))
GOLD_Q = np.load(os.path.join(HERE, "golden", "golden_quantizer.npz"))
_cuda_path = os.path.join(HERE, "golden", "golden_reference_cuda.npz")
GOLD_C = np.load(_cuda_path) if os.path.exists(_cuda_path) else None
needs_cuda_golden = pytest.mark.skipif(GOLD_C is None, reason="golden_reference_cuda.npz not generated yet")

CASES = list(range(len(QUANT_CASES)))


@pytest.mark.parametrize("i", CASES)
def test_quantizer_matches_reference_python(i):
    N, K, g, seed, std = QUANT_CASES[i]
    w = seeded_weight(N, K, seed, std)
    qweight, zeros, scales, w_fp16 = oracle.generate_quant(w, 4, g)
    assert np.array_equal(qweight.numpy(), GOLD_Q[f"c{i}_qweight"])
    assert np.array_equal(zeros.numpy().view(np.uint16), GOLD_Q[f"c{i}_zeros"])
    assert np.array_equal(scales.numpy().view(np.uint16), GOLD_Q[f"c{i}_scales"])
    assert np.array_equal(w_fp16.numpy().view(np.uint16), GOLD_Q[f"c{i}_wfp16"])


@pytest.mark.parametrize("i", CASES)
def test_closed_form_address_matches_literal_permutation(i):
    """unpack() uses the closed-form element address; pack() the literal 10-D permutation."""
    N, K, g, seed, std = QUANT_CASES[i]
    qw8 = GOLD_Q[f"c{i}_qweight"]
    awq = oracle.convert_ours_to_awq(qw8, K, N)
    packed = oracle.convert_awq_to_lmdeploy(awq, K, N)
    q = oracle.unpack(packed, K, N)
    expect = np.empty((N, K), dtype=np.uint8)
    expect[:, 0::2] = qw8 >> 4
    expect[:, 1::2] = qw8 & 0xF
    assert np.array_equal(q, expect)


@pytest.mark.parametrize("i", CASES)
def test_dequant_equals_quantizer_w_fp16(i):
    """dequant(packed) == the quantizer's own (q - zeros) * scales bit for bit, except where the
    kernel's flush-to-zero bites (denormal scale or product): there the oracle yields 0."""
    N, K, g, seed, std = QUANT_CASES[i]
    packed, zs = oracle.pack(GOLD_Q[f"c{i}_qweight"], GOLD_Q[f"c{i}_zeros"], GOLD_Q[f"c{i}_scales"], K, N, g)
    w = oracle.dequant(packed, zs, K, N, g).view(np.uint16)
    gold = GOLD_Q[f"c{i}_wfp16"]
    scales = np.repeat(GOLD_Q[f"c{i}_scales"], g, axis=1)
    sub = ((scales >> 10) & 0x1F) == 0                 # denormal (or zero) scale
    assert np.array_equal(w[~sub], gold[~sub])
    assert np.all((w[sub] & 0x7FFF) == 0)
    if std > 1e-3:
        assert not sub.any()
    else:
        assert sub.any()                               # the crafted case really reaches the FTZ regime


@needs_cuda_golden
@pytest.mark.parametrize("i", CASES)
def test_layout_matches_reference_cuda(i):
    N, K, g, seed, std = QUANT_CASES[i]
    zs = oracle.transpose_merge_zeros_scales(GOLD_Q[f"c{i}_zeros"], GOLD_Q[f"c{i}_scales"], K, N, g)
    assert np.array_equal(zs, GOLD_C[f"c{i}_zs"])
    awq = oracle.convert_ours_to_awq(GOLD_Q[f"c{i}_qweight"], K, N)
    assert np.array_equal(awq.view(np.uint8).reshape(K, N // 2), GOLD_C[f"c{i}_awq"])
    lmd = oracle.convert_awq_to_lmdeploy(awq, K, N)
    assert np.array_equal(lmd.view(np.int32), GOLD_C[f"c{i}_lmdeploy"])


@needs_cuda_golden
@pytest.mark.parametrize("i", CASES)
def test_dequant_matches_reference_kernel_identity_trick(i):
    if f"c{i}_identity" not in GOLD_C:
        pytest.skip("reference kernel has no tile config for this case")
    N, K, g, seed, std = QUANT_CASES[i]
    w = oracle.dequant(GOLD_C[f"c{i}_lmdeploy"], GOLD_C[f"c{i}_zs"], K, N, g).view(np.uint16)
    ref = GOLD_C[f"c{i}_identity"]
    # -0 vs +0 cannot be told apart through a GEMM (0 * 1 + 0 ...): compare modulo the sign of zero
    wz, rz = w.copy(), ref.copy()
    wz[(wz & 0x7FFF) == 0] = 0
    rz[(rz & 0x7FFF) == 0] = 0
    assert np.array_equal(wz, rz)


def _self_consistent_rows(ref, x, w_ident, K):
    """Rows of a reference-kernel output that agree with the reference's OWN dequantised weight
    (read back through its identity-matrix GEMM) multiplied in float64.  Rebuilt unmodified for
    sm_100a, the reference kernel returns wrong token rows for some of its tile configurations
    (observed: N=256 K=512, tokens 16 -> rows 0-7, tokens 40 -> rows 0-31); those rows cannot pin
    anything and are excluded - and counted."""
    truth = x[0].double().numpy() @ w_ident.astype(np.float64).T
    bound = 1e-2 * float(x.abs().max()) * np.sqrt(K) * float(np.abs(w_ident.astype(np.float32)).max())
    return np.abs(ref.astype(np.float64) - truth).max(axis=1) <= bound


@needs_cuda_golden
@pytest.mark.parametrize("i", CASES)
def test_gemm_within_tolerance_of_reference_kernel(i):
    if f"c{i}_gemm_m1" not in GOLD_C:
        pytest.skip("reference kernel has no tile config for this case")
    N, K, g, seed, std = QUANT_CASES[i]
    w = oracle.dequant(GOLD_C[f"c{i}_lmdeploy"], GOLD_C[f"c{i}_zs"], K, N, g)
    w_ident = GOLD_C[f"c{i}_identity"].view(np.float16)
    checked = 0
    for M in GEMM_TOKENS:
        x = seeded_x(M, K, seed)
        mine = oracle.gemm_f16(x, w).astype(np.float32)
        ref = GOLD_C[f"c{i}_gemm_m{M}"].view(np.float16).astype(np.float32)
        ok = _self_consistent_rows(ref, x, w_ident, K)
        # the oracle itself must be consistent on every row
        assert _self_consistent_rows(mine, x, w_ident, K).all()
        if ok.any():
            check_gemm_tolerance(mine[ok], ref[ok], x, w, K)
            checked += int(ok.sum())
    assert checked >= sum(GEMM_TOKENS) // 3


@needs_cuda_golden
def test_reference_kernel_bad_rows_are_the_known_ones():
    """Documents (and bounds) where the rebuilt reference kernel disagrees with its own weights."""
    bad = {}
    for i, (N, K, g, seed, std) in enumerate(QUANT_CASES):
        if f"c{i}_gemm_m1" not in GOLD_C:
            continue
        w_ident = GOLD_C[f"c{i}_identity"].view(np.float16)
        for M in GEMM_TOKENS:
            ref = GOLD_C[f"c{i}_gemm_m{M}"].view(np.float16).astype(np.float32)
            ok = _self_consistent_rows(ref, seeded_x(M, K, seed), w_ident, K)
            if not ok.all():
                bad[(N, K, M)] = np.where(~ok)[0].tolist()
    assert set(bad) <= {(256, 512, 16), (256, 512, 40)}, bad


def test_fp16_primitives_against_torch():
    L = oracle.lib()
    g = torch.Generator().manual_seed(5)
    a = (torch.randn(4000, generator=g) * torch.pow(10.0, torch.randint(-7, 4, (4000,), generator=g).float())).half()
    b = torch.randn(4000, generator=g).half()
    au, bu = a.numpy().view(np.uint16), b.numpy().view(np.uint16)
    add = np.array([L.oracle_hadd(int(x), int(y)) for x, y in zip(au, bu)], dtype=np.uint16)
    assert np.array_equal(add, (a + b).numpy().view(np.uint16))
    f = torch.randn(4000, generator=g) * 300
    fh = np.array([L.oracle_f2h(float(v)) for v in f], dtype=np.uint16)
    assert np.array_equal(fh, f.half().numpy().view(np.uint16))
    # mul with FTZ: equals torch's product wherever neither input nor result is subnormal
    mul = np.array([L.oracle_hmul_ftz(int(x), int(y)) for x, y in zip(au, bu)], dtype=np.uint16)
    ref = (a * b).numpy().view(np.uint16)
    normal = lambda u: ((u >> 10) & 0x1F) != 0
    ok = normal(au) & normal(bu) & normal(ref)
    assert np.array_equal(mul[ok], ref[ok])
    sub_in = ~normal(au) | ~normal(bu)
    assert np.all((mul[sub_in] & 0x7FFF) == 0)


def test_gemm_restated_numerics():
    g = torch.Generator().manual_seed(9)
    x = torch.randn(7, 256, generator=g).half()
    w = (torch.randn(48, 256, generator=g) * 0.05).half()
    bias = (torch.randn(48, generator=g) * 0.1).half()
    out = oracle.gemm_f16(x, w, bias)
    ref = (x.double() @ w.double().t()).float().half() + bias          # fp16 add after fp16 rounding
    diff = (torch.from_numpy(out.astype(np.float32)) - ref.float()).abs().max().item()
    assert diff <= 2e-3
