"""Drop-in check with the reference's OWN Python on top of this library's `quant` module.

oracle/build_ref.py stages the reference's WALinear (test/nvidia/module/qlinear/qlinear.py) and quantizer
(test/nvidia/utils/quant_dequant_nvidia.py, quant_funcs.py) unmodified under oracle/_ref/refpy/.  Here they are
imported with sparse-quant_b200/ on sys.path, so that their `from quant import ...` lines bind to this library:
`from_float` (quantise + the three layout kernels), `forward` (gemm_awq_ut + the module's own bias add) and
`state_dict()` run exactly as the reference's model builder runs them (test/nvidia/opt_infer.py:86-89).  Checked
against the oracle, and a state dict saved by the reference's module must load into this package's WALinear and
give the same outputs.  Skipped when the staged files are absent."""
import importlib
import os
import sys

import numpy as np
import pytest
import torch

import oracle
from helpers import check_gemm_tolerance

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REFPY = os.path.join(ROOT, "oracle", "_ref", "refpy")


@pytest.fixture(scope="module")
def ref_walinear():
    if not os.path.exists(os.path.join(REFPY, "module", "qlinear", "qlinear.py")):
        pytest.skip("reference Python not staged (oracle/build_ref.py needs the reference tree)")
    import quant                                             # this library's module must be the one they bind to
    assert os.path.dirname(quant.__file__).startswith(os.path.join(ROOT, "sparse-quant_b200"))
    saved = {k: sys.modules.pop(k) for k in list(sys.modules) if k == "utils" or k.startswith("utils.") or k == "module" or k.startswith("module.")}
    sys.path.insert(0, REFPY)
    try:
        mod = importlib.import_module("module.qlinear.qlinear")
        yield mod.WALinear
    finally:
        sys.path.remove(REFPY)
        for k in [k for k in sys.modules if k == "utils" or k.startswith("utils.") or k == "module" or k.startswith("module.")]:
            del sys.modules[k]
        sys.modules.update(saved)


@pytest.mark.parametrize("K,N,bias", [(512, 256, True), (1024, 384, False), (4096, 4096, True)])
def test_reference_walinear_runs_on_this_quant_module(ref_walinear, K, N, bias):
    from w4a16 import WALinear
    g = 128
    torch.manual_seed(K + N)
    lin = torch.nn.Linear(K, N, bias=bias).half().cuda()
    lin.weight.data.mul_(0.02 / lin.weight.data.float().std().item())           # N(0, 0.02)-like spread
    w_cpu = lin.weight.data.cpu().clone()
    b_cpu = lin.bias.data.cpu().clone().unsqueeze(0) if bias else None
    q = ref_walinear.from_float(lin, {"n_bit": 4, "group_size": g}, None)        # the reference's own packing flow
    assert repr(q) == f"W4A16Linear({K}, {N})"
    o_qw, o_zs, _ = oracle.quant_pack(w_cpu, g)
    assert q.weight.dtype == torch.int32 and tuple(q.weight.shape) == (K, N // 8)
    assert np.array_equal(q.weight.cpu().numpy().view(np.uint32), o_qw), "packed weight differs from the oracle"
    assert np.array_equal(q.zeros_scales.cpu().numpy().view(np.uint16), o_zs), "zeros_scales differs from the oracle"
    w_deq = oracle.dequant(o_qw, o_zs, K, N, g)

    for shape in [(1, 1, K), (2, 3, K), (1, 40, K)]:                              # decode kernels and the tcgen05 kernel
        x = torch.randn(*shape, dtype=torch.float16, device="cuda")
        y = q(x)                                                                 # gemm_awq_ut + `y + self.bias` ([1, N] on 3-D)
        torch.cuda.synchronize()
        assert tuple(y.shape) == (shape[0], shape[1], N) and y.dtype == torch.float16
        ref = oracle.gemm_f16(x.cpu().reshape(1, -1, K), w_deq, b_cpu).astype(np.float32)
        check_gemm_tolerance(y.reshape(-1, N), ref, x, w_deq, K)

    # a state dict written by the reference's module loads into this package's module: same keys, same outputs
    sd = q.state_dict()
    assert set(sd) == ({"zeros_scales", "weight", "bias"} if bias else {"zeros_scales", "weight"})
    mine = WALinear(K, N, w_bit=4, group_size=g, bias=bias)
    mine.load_state_dict(sd)
    x = torch.randn(2, 5, K, dtype=torch.float16, device="cuda")
    assert torch.equal(mine(x), q(x))      # the fused bias add rounds exactly like the module's separate fp16 add


@pytest.mark.parametrize("kind", ["opt", "llama"])
def test_state_dict_written_by_the_reference_modules_runs_on_the_gpu(ref_walinear, kind, tmp_path, monkeypatch):
    """Checkpoint I/O on the reference's own output: every linear of a small OPT- / LLaMA-shaped model is quantised
    by the reference's WALinear.from_float, its state_dict() entries are filed under the Hugging Face parameter names
    the reference's save_pretrained uses (test/nvidia/opt_infer.py:86-89), written with torch.save, read back and
    loaded into this package's decoder stack on the GPU.  Prefill logits and greedily decoded tokens must agree with
    the same state dict run on the CPU with the oracle standing in for the kernels."""
    import w4a16.qlinear as ql
    from test_tp_cpu import _oracle_forward
    from w4a16.checkpoint import decoder_from_state_dict
    from w4a16.models import DecoderConfig
    g = 128
    if kind == "opt":
        cfg = DecoderConfig("opt", layers=2, hidden=256, heads=4, ffn=512, vocab=96, group_size=g, max_positions=48)
    else:
        cfg = DecoderConfig("llama", layers=2, hidden=256, heads=4, ffn=384, vocab=96, group_size=g, max_positions=48)
    H, F = cfg.hidden, cfg.ffn
    gen = torch.Generator().manual_seed(17)
    sd = {}

    def lin(prefix, K, N, bias):
        m = torch.nn.Linear(K, N, bias=bias).half()
        m.weight.data = (torch.randn(N, K, generator=gen) * 0.05).half()
        if bias:
            m.bias.data = (torch.randn(N, generator=gen) * 0.05).half()
        q = ref_walinear.from_float(m.cuda(), {"n_bit": 4, "group_size": g}, None)
        for k, v in q.state_dict().items():
            sd[f"{prefix}.{k}"] = v.detach().cpu().clone()

    def vec(key, n, base=0.0):
        sd[key] = (base + 0.1 * torch.randn(n, generator=gen)).half()

    if kind == "opt":
        sd["model.decoder.embed_tokens.weight"] = (torch.randn(cfg.vocab, H, generator=gen) * 0.05).half()
        sd["model.decoder.embed_positions.weight"] = (torch.randn(cfg.max_positions + 2, H, generator=gen) * 0.05).half()
        sd["lm_head.weight"] = sd["model.decoder.embed_tokens.weight"]
        for i in range(cfg.layers):
            p = f"model.decoder.layers.{i}."
            for n in ("q_proj", "k_proj", "v_proj", "out_proj"):
                lin(p + "self_attn." + n, H, H, True)
            lin(p + "fc1", H, F, True)
            lin(p + "fc2", F, H, True)
            for n in ("self_attn_layer_norm", "final_layer_norm"):
                vec(p + n + ".weight", H, 1.0)
                vec(p + n + ".bias", H)
        vec("model.decoder.final_layer_norm.weight", H, 1.0)
        vec("model.decoder.final_layer_norm.bias", H)
    else:
        sd["model.embed_tokens.weight"] = (torch.randn(cfg.vocab, H, generator=gen) * 0.05).half()
        sd["lm_head.weight"] = (torch.randn(cfg.vocab, H, generator=gen) * 0.05).half()
        for i in range(cfg.layers):
            p = f"model.layers.{i}."
            for n in ("q_proj", "k_proj", "v_proj", "o_proj"):
                lin(p + "self_attn." + n, H, H, False)
            lin(p + "mlp.gate_proj", H, F, False)
            lin(p + "mlp.up_proj", H, F, False)
            lin(p + "mlp.down_proj", F, H, False)
            vec(p + "input_layernorm.weight", H, 1.0)
            vec(p + "post_attention_layernorm.weight", H, 1.0)
        vec("model.norm.weight", H, 1.0)
    path = tmp_path / "pytorch_model.bin"
    torch.save(sd, path)
    loaded = torch.load(path)

    ids = torch.randint(0, cfg.vocab, (3, 9), generator=torch.Generator().manual_seed(2))
    gpu = decoder_from_state_dict(cfg, loaded, 0, 1, None, "cuda").mark_static()
    gpu.reset(3, 24)
    logits_gpu = gpu(ids.cuda()).float().cpu()
    tokens_gpu, _, _ = gpu.generate_graphed(ids.cuda(), 6, use_graph=True)          # decode kernels, attention, fused epilogues

    monkeypatch.setattr(ql, "gemm_awq_bias", _oracle_forward)                        # the CPU run: oracle instead of kernels
    cpu = decoder_from_state_dict(cfg, loaded, 0, 1, None, "cpu")
    cpu.reset(3, 24)
    logits_cpu = cpu(ids).float()
    scale = float(logits_cpu.abs().max())
    assert float((logits_gpu - logits_cpu).abs().max()) <= 2e-2 * max(scale, 1.0)
    # greedy continuation: the first new token is the arg-max of those logits wherever the margin is not a tie
    top2 = logits_cpu.topk(2, dim=-1).values
    clear = (top2[:, 0] - top2[:, 1]) > 4e-2 * max(scale, 1.0)
    assert torch.equal(tokens_gpu[:, 0].cpu()[clear], logits_cpu.argmax(-1)[clear])
    assert tokens_gpu.shape == (3, 6) and int(tokens_gpu.min()) >= 0 and int(tokens_gpu.max()) < cfg.vocab
