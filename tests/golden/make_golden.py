#!/usr/bin/env python3
"""Generate the golden vectors under tests/golden/ from the REFERENCE itself.

  --cpu   (any machine with the reference tree): imports the reference's own Python quantizer
          (test/nvidia/utils/quant_dequant_nvidia.py, with a stub in place of its CUDA extension)
          and records, for seeded weights, what generate_quant returns -> golden_quantizer.npz
  --gpu   (a B200 with oracle/_ref built by oracle/build_ref.py): runs the reference's own CUDA
          extension (transpose_merge_zeros_scales, convert_ours_to_awq, convert_awq_to_lmdeploy,
          gemm_awq_ut incl. the identity-matrix trick that reads back its in-kernel dequant) on the
          vectors of --cpu -> <out>/golden_reference_cuda.npz (copy it to tests/golden/).

The inputs are regenerated from seeds (torch CPU generator), so the two stages agree.
"""
import argparse
import importlib.util
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))

# (N, K, g, seed, std)
QUANT_CASES = [
    (64, 128, 128, 11, 0.02),
    (96, 256, 64, 12, 0.02),
    (32, 128, 32, 13, 0.5),
    (128, 256, 128, 14, 0.02),
    (256, 512, 128, 15, 0.02),
    (64, 256, 128, 16, 1e-7),     # constant-ish groups: scale clamps to a denormal -> FTZ regime
]
GEMM_TOKENS = [1, 5, 16, 40]      # for the g=128 cases the reference kernel can run


def seeded_weight(N, K, seed, std):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(N, K, generator=g) * std).half()


def seeded_x(M, K, seed):
    g = torch.Generator().manual_seed(1000 + seed)
    return torch.randn(1, M, K, generator=g).half()


def cpu_stage(reference):
    stub = types.ModuleType("quant")
    for n in ("transpose_merge_zeros_scales", "convert_ours_to_awq", "convert_awq_to_lmdeploy", "gemm_awq_ut"):
        setattr(stub, n, None)
    sys.modules["quant"] = stub
    spec = importlib.util.spec_from_file_location(
        "ref_quant_dequant", os.path.join(reference, "test", "nvidia", "utils", "quant_dequant_nvidia.py"))
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    out = {}
    for i, (N, K, g, seed, std) in enumerate(QUANT_CASES):
        w = seeded_weight(N, K, seed, std)
        qweight, zeros, scales, w_fp16 = ref.generate_quant(w, K, 4, g)
        out[f"c{i}_shape"] = np.array([N, K, g, seed], dtype=np.int64)
        out[f"c{i}_std"] = np.array([std])
        out[f"c{i}_qweight"] = qweight.numpy()
        out[f"c{i}_zeros"] = zeros.numpy().view(np.uint16)
        out[f"c{i}_scales"] = scales.numpy().view(np.uint16)
        out[f"c{i}_wfp16"] = w_fp16.numpy().view(np.uint16)
    path = os.path.join(HERE, "golden_quantizer.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


def gpu_stage(out_dir):
    so = [f for f in os.listdir(os.path.join(ROOT, "oracle", "_ref")) if f.startswith("quant") and f.endswith(".so")]
    spec = importlib.util.spec_from_file_location("quant", os.path.join(ROOT, "oracle", "_ref", so[0]))
    refq = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(refq)
    gold = np.load(os.path.join(HERE, "golden_quantizer.npz"))
    out = {}
    dev = "cuda"
    for i, (N, K, g, seed, std) in enumerate(QUANT_CASES):
        qweight = torch.from_numpy(gold[f"c{i}_qweight"]).to(dev)
        zeros = torch.from_numpy(gold[f"c{i}_zeros"].view(np.float16)).to(dev)
        scales = torch.from_numpy(gold[f"c{i}_scales"].view(np.float16)).to(dev)
        zs = torch.empty((K // g, 2 * N), dtype=torch.float16, device=dev)
        refq.transpose_merge_zeros_scales(zeros, scales, zs, K, N, g)
        awq = torch.empty((K, N // 2), dtype=torch.uint8, device=dev)
        refq.convert_ours_to_awq(qweight, awq, K, N)
        lmd = torch.empty((K, N // 8), dtype=torch.int32, device=dev)
        refq.convert_awq_to_lmdeploy(awq, lmd, K, N)
        torch.cuda.synchronize()
        out[f"c{i}_zs"] = zs.cpu().numpy().view(np.uint16)
        out[f"c{i}_awq"] = awq.cpu().numpy()
        out[f"c{i}_lmdeploy"] = lmd.cpu().numpy()
        # the reference kernel only instantiates g=128 and needs (N%128==0 and K%32==0) or (N%64==0 and K%256==0)
        if g == 128 and ((N % 128 == 0) or (N % 64 == 0 and K % 256 == 0)):
            eye = torch.eye(K, dtype=torch.float16, device=dev).unsqueeze(0)
            o = refq.gemm_awq_ut(eye, lmd, zs, K, N, K, g)
            torch.cuda.synchronize()
            out[f"c{i}_identity"] = o[0].t().contiguous().cpu().numpy().view(np.uint16)   # [N, K] = in-kernel dequant
            for M in GEMM_TOKENS:
                x = seeded_x(M, K, seed).to(dev)
                o = refq.gemm_awq_ut(x, lmd, zs, M, N, K, g)
                torch.cuda.synchronize()
                out[f"c{i}_gemm_m{M}"] = o[0].cpu().numpy().view(np.uint16)
    os.makedirs(out_dir, exist_ok=True)
    path = os.path.join(out_dir, "golden_reference_cuda.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--cpu", action="store_true")
    ap.add_argument("--gpu", action="store_true")
    ap.add_argument("--reference", default=os.environ.get("W4A16_REFERENCE") or os.path.join(os.path.dirname(ROOT), "reference"),
                    help="checkout of the reference project (CPU stage only)")
    ap.add_argument("--out", default=os.path.join(ROOT, "tests", "golden"),
                    help="directory that receives golden_reference_cuda.npz (GPU stage)")
    a = ap.parse_args()
    if a.cpu:
        cpu_stage(a.reference)
    if a.gpu:
        gpu_stage(a.out)
