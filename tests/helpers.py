"""Shared helpers of the test-suite (seeded synthetic inputs, tolerances)."""
import math

import numpy as np
import torch

import oracle


def make_weight(N, K, seed=1234, std=0.02):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(N, K, generator=g) * std).half()


def make_x(M, K, seed=4321, std=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(1, M, K, generator=g) * std).half()


def make_packed(N, K, g, seed=1234):
    """-> dict with qweight uint32 [K,N/8], zs uint16 [K/g,2N], w_fp16 (torch fp16 [N,K], the
    quantizer's own dequantised weight), w_deq (np.float16 [N,K], oracle dequant of the packed tensors)."""
    w = make_weight(N, K, seed)
    qweight, zs, w_fp16 = oracle.quant_pack(w, g)
    return dict(N=N, K=K, g=g, qweight=qweight, zs=zs, w_fp16=w_fp16,
                w_deq=oracle.dequant(qweight, zs, K, N, g))


def to_dev(p, device="cuda"):
    qw = torch.from_numpy(p["qweight"].view(np.int32)).to(device)
    zs = torch.from_numpy(p["zs"].view(np.float16)).to(device)
    return qw, zs


def check_gemm_tolerance(out, ref, x, w_deq, K):
    """north_star tolerance: max|err| <= 1e-2 * |x|inf * sqrt(K) * max|w| and relative
    Frobenius error <= 2e-3 against dequantise-then-matmul; plus the reference script's
    allclose(atol=2e-2, rtol=2e-2) floor (quantization/nvidia/script/gemm_awq_test.py:105)."""
    out = torch.as_tensor(np.asarray(out, dtype=np.float32)) if not torch.is_tensor(out) else out.float().cpu()
    ref = torch.as_tensor(np.asarray(ref, dtype=np.float32)) if not torch.is_tensor(ref) else ref.float().cpu()
    out = out.reshape(ref.shape)
    xmax = float(torch.as_tensor(np.asarray(x, dtype=np.float32)).abs().max()) if not torch.is_tensor(x) else float(x.float().abs().max())
    wmax = float(np.abs(np.asarray(w_deq, dtype=np.float32)).max())
    bound = 1e-2 * xmax * math.sqrt(K) * wmax
    err = (out - ref).abs().max().item()
    fro = ((out - ref).norm() / ref.norm().clamp_min(1e-12)).item()
    assert err <= bound + 1e-6, f"max abs err {err} > bound {bound}"
    assert fro <= 2e-3, f"relative Frobenius error {fro} > 2e-3"
    assert torch.allclose(out, ref, atol=2e-2, rtol=2e-2)
    return err, fro


def check_gemm_sampled(out, x, p, bias=None, n_tok=16, n_out=48, seed=99):
    """The same tolerances on a seeded sample of token rows x out-feature columns (>= 256 outputs), for problems
    whose full oracle product would take minutes on the CPU: out torch [M, N] (device), x torch fp16 [1, M, K],
    p a make_packed() dict, bias torch fp16 [1, N] or None."""
    rng = np.random.default_rng(seed)
    M, N = out.shape
    toks = np.sort(rng.choice(M, size=min(n_tok, M), replace=False))
    cols = np.sort(rng.choice(N, size=min(n_out, N), replace=False))
    xs = x[:, torch.from_numpy(toks)].contiguous()
    ws = np.ascontiguousarray(p["w_deq"][cols])
    bs = None if bias is None else bias[:, torch.from_numpy(cols)].contiguous()
    ref = oracle.gemm_f16(xs, ws, bs).astype(np.float32)
    got = out[torch.from_numpy(toks).to(out.device)][:, torch.from_numpy(cols).to(out.device)]
    # the bound uses the norms of the whole problem, as the full check does
    xmax = float(x.float().abs().max())
    wmax = float(np.abs(p["w_deq"].astype(np.float32)).max())
    got = got.float().cpu()
    ref_t = torch.from_numpy(ref).reshape(got.shape)
    err = (got - ref_t).abs().max().item()
    fro = ((got - ref_t).norm() / ref_t.norm().clamp_min(1e-12)).item()
    assert err <= 1e-2 * xmax * math.sqrt(p["K"]) * wmax + 1e-6, f"max abs err {err}"
    assert fro <= 2e-3, f"relative Frobenius error {fro} > 2e-3"
    assert torch.allclose(got, ref_t, atol=2e-2, rtol=2e-2)
    return err, fro
