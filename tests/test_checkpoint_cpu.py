"""Reference-format checkpoints (Hugging Face module names, WALinear buffers `weight` / `zeros_scales` / `bias`) loaded
into the decoder stacks, on CPU: key mapping for both architectures, torch.save/torch.load round trip, exact sharding
and packed-domain fusion of the loaded tensors, and the error messages for malformed entries."""
import numpy as np
import pytest
import torch

import oracle
from helpers import make_weight
from test_tp_cpu import _oracle_forward


def _cfg(kind):
    from w4a16.models import DecoderConfig
    if kind == "opt":
        return DecoderConfig("opt", layers=2, hidden=256, heads=4, ffn=512, vocab=96, group_size=128, max_positions=32)
    return DecoderConfig("llama", layers=2, hidden=256, heads=4, ffn=320, vocab=96, group_size=64, max_positions=32)


def _packed(N, K, g, seed):
    qw, zs, _ = oracle.quant_pack(make_weight(N, K, seed), g)
    return torch.from_numpy(qw.view(np.int32).copy()), torch.from_numpy(zs.view(np.float16).copy())


def _reference_state_dict(cfg, seed=3):
    """What the reference's save_pretrained would hold for a model of this shape (random contents)."""
    gen = torch.Generator().manual_seed(seed)
    H, F, g = cfg.hidden, cfg.ffn, cfg.group_size
    sd = {}

    def lin(prefix, K, N, s, bias):
        sd[prefix + ".weight"], sd[prefix + ".zeros_scales"] = _packed(N, K, g, s)
        if bias:
            sd[prefix + ".bias"] = (torch.randn(1, N, generator=gen) * 0.05).half()

    def vec(key, n, base=0.0):
        sd[key] = (base + 0.1 * torch.randn(n, generator=gen)).half()

    if cfg.kind == "opt":
        sd["model.decoder.embed_tokens.weight"] = (torch.randn(cfg.vocab, H, generator=gen) * 0.02).half()
        sd["model.decoder.embed_positions.weight"] = (torch.randn(cfg.max_positions + 2, H, generator=gen) * 0.02).half()
        sd["lm_head.weight"] = sd["model.decoder.embed_tokens.weight"]
        for i in range(cfg.layers):
            p = f"model.decoder.layers.{i}."
            for j, n in enumerate(("q_proj", "k_proj", "v_proj", "out_proj")):
                lin(p + "self_attn." + n, H, H, 10 * i + j, True)
            lin(p + "fc1", H, F, 10 * i + 4, True)
            lin(p + "fc2", F, H, 10 * i + 5, True)
            for n in ("self_attn_layer_norm", "final_layer_norm"):
                vec(p + n + ".weight", H, 1.0)
                vec(p + n + ".bias", H)
        vec("model.decoder.final_layer_norm.weight", H, 1.0)
        vec("model.decoder.final_layer_norm.bias", H)
    else:
        sd["model.embed_tokens.weight"] = (torch.randn(cfg.vocab, H, generator=gen) * 0.02).half()
        sd["lm_head.weight"] = (torch.randn(cfg.vocab, H, generator=gen) * 0.02).half()
        for i in range(cfg.layers):
            p = f"model.layers.{i}."
            for j, n in enumerate(("q_proj", "k_proj", "v_proj", "o_proj")):
                lin(p + "self_attn." + n, H, H, 10 * i + j, False)
            lin(p + "mlp.gate_proj", H, F, 10 * i + 4, False)
            lin(p + "mlp.up_proj", H, F, 10 * i + 5, False)
            lin(p + "mlp.down_proj", F, H, 10 * i + 6, False)
            vec(p + "input_layernorm.weight", H, 1.0)
            vec(p + "post_attention_layernorm.weight", H, 1.0)
        vec("model.norm.weight", H, 1.0)
    return sd


def _deq(w, zs, K, N, g):
    return oracle.dequant(w.numpy().view(np.uint32), zs.numpy().view(np.uint16), K, N, g)


@pytest.mark.parametrize("kind", ["opt", "llama"])
def test_checkpoint_loads_shards_and_fuses_exactly(kind, tmp_path, monkeypatch):
    import w4a16.qlinear as ql
    from w4a16.checkpoint import decoder_from_state_dict
    cfg = _cfg(kind)
    sd = _reference_state_dict(cfg)
    path = tmp_path / "pytorch_model.bin"
    torch.save(sd, path)
    sd = torch.load(path)
    H, F, g = cfg.hidden, cfg.ffn, cfg.group_size
    lp = "model.decoder.layers.1." if kind == "opt" else "model.layers.1."
    full_q = _deq(sd[lp + "self_attn.q_proj.weight"], sd[lp + "self_attn.q_proj.zeros_scales"], H, H, g)
    full_k = _deq(sd[lp + "self_attn.k_proj.weight"], sd[lp + "self_attn.k_proj.zeros_scales"], H, H, g)
    full_v = _deq(sd[lp + "self_attn.v_proj.weight"], sd[lp + "self_attn.v_proj.zeros_scales"], H, H, g)
    out_name = "self_attn.out_proj" if kind == "opt" else "self_attn.o_proj"
    full_o = _deq(sd[lp + out_name + ".weight"], sd[lp + out_name + ".zeros_scales"], H, H, g)
    for world in (1, 2):
        for rank in range(world):
            m = decoder_from_state_dict(cfg, sd, rank, world, None, "cpu")
            layer = m.layers[1]
            n0, n1 = rank * H // world, (rank + 1) * H // world
            qkv = layer.qkv_proj
            got = _deq(qkv.weight, qkv.zeros_scales, H, 3 * (n1 - n0), g)
            want = np.concatenate([full_q[n0:n1], full_k[n0:n1], full_v[n0:n1]], axis=0)
            assert np.array_equal(got.view(np.uint16), want.view(np.uint16))
            o = layer.out_proj.linear
            got_o = _deq(o.weight, o.zeros_scales, n1 - n0, H, g)
            assert np.array_equal(got_o.view(np.uint16), full_o[:, n0:n1].view(np.uint16))
            if kind == "opt":
                assert torch.equal(qkv.bias[0, :n1 - n0], sd[lp + "self_attn.q_proj.bias"][0, n0:n1])
                assert torch.equal(layer.ln1.weight, sd[lp + "self_attn_layer_norm.weight"])
                assert torch.equal(layer.ln2.bias, sd[lp + "final_layer_norm.bias"])
                assert torch.equal(m.pos_embed, sd["model.decoder.embed_positions.weight"])
                assert torch.equal(m.final_norm.weight, sd["model.decoder.final_layer_norm.weight"])
            else:
                assert qkv.bias is None
                assert torch.equal(layer.ln1.weight, sd[lp + "input_layernorm.weight"])
                assert torch.equal(m.final_norm.weight, sd["model.norm.weight"])
                gu = layer.gate_up_proj
                assert gu.out_features == 2 * (layer.fc2.k1 - layer.fc2.k0)
            v0, v1 = m.vocab_ranges[rank]
            assert torch.equal(m.lm_head, sd["lm_head.weight"][v0:v1])
    # the loaded single-rank model runs (the CPU oracle stands in for the kernel)
    monkeypatch.setattr(ql, "gemm_awq_bias", _oracle_forward)
    m = decoder_from_state_dict(cfg, sd, 0, 1, None, "cpu")
    m.reset(2, 8)
    logits = m(torch.randint(0, cfg.vocab, (2, 5), generator=torch.Generator().manual_seed(1)))
    assert logits.shape == (2, cfg.vocab) and torch.isfinite(logits.float()).all()


def test_checkpoint_errors_name_the_entry():
    from w4a16.checkpoint import decoder_from_state_dict
    cfg = _cfg("opt")
    sd = _reference_state_dict(cfg)
    bad = dict(sd)
    del bad["model.decoder.layers.0.fc1.zeros_scales"]
    with pytest.raises(KeyError, match="fc1.zeros_scales"):
        decoder_from_state_dict(cfg, bad, 0, 1, None, "cpu")
    bad = dict(sd)
    bad["model.decoder.layers.0.fc2.weight"] = bad["model.decoder.layers.0.fc2.weight"][:, :4]
    with pytest.raises(ValueError, match="fc2.weight"):
        decoder_from_state_dict(cfg, bad, 0, 1, None, "cpu")
    bad = dict(sd)
    bad["model.decoder.layers.1.self_attn.q_proj.weight"] = bad["model.decoder.layers.1.self_attn.q_proj.weight"].float()
    with pytest.raises(TypeError, match="q_proj.weight"):
        decoder_from_state_dict(cfg, bad, 0, 1, None, "cpu")
