"""Loading a model that the reference quantised and saved into the decoder stacks of w4a16.models.

The reference replaces every nn.Linear of a Hugging Face OPT / LLaMA model (except lm_head) by its WALinear
(test/nvidia/quantizer/opt_quantizer.py:12-23, llama_quantizer.py) and saves with save_pretrained
(test/nvidia/opt_infer.py:86-89).  The state dict therefore keeps the Hugging Face module names, and every quantised
linear contributes three entries (test/nvidia/module/qlinear/qlinear.py:26-34):

    <prefix>.weight        int32 [K, N/8]   packed, tile-ordered
    <prefix>.zeros_scales  fp16  [K/g, 2N]  interleaved (zero + 64, scale)
    <prefix>.bias          fp16  [1, N]     (OPT only)

StateDictSource hands those tensors to w4a16.models.Decoder, which shards them for its rank (exact slices of the
packed tensors, no re-quantisation) and fuses q/k/v and gate/up in the packed domain.  Layers quantised with
w_bit=2 are not supported (WALinear raises for them).
"""
from __future__ import annotations

import torch
from torch import nn

from .models import Decoder, DecoderConfig, RMSNorm
from .qlinear import WALinear

_OPT = {
    "layer": "model.decoder.layers.{i}.",
    "q_proj": "self_attn.q_proj", "k_proj": "self_attn.k_proj", "v_proj": "self_attn.v_proj", "out_proj": "self_attn.out_proj",
    "fc1": "fc1", "fc2": "fc2", "ln1": "self_attn_layer_norm", "ln2": "final_layer_norm",
    "final": "model.decoder.final_layer_norm", "embed": "model.decoder.embed_tokens.weight",
    "pos_embed": "model.decoder.embed_positions.weight", "lm_head": "lm_head.weight",
}
_LLAMA = {
    "layer": "model.layers.{i}.",
    "q_proj": "self_attn.q_proj", "k_proj": "self_attn.k_proj", "v_proj": "self_attn.v_proj", "out_proj": "self_attn.o_proj",
    "gate_proj": "mlp.gate_proj", "up_proj": "mlp.up_proj", "down_proj": "mlp.down_proj",
    "ln1": "input_layernorm", "ln2": "post_attention_layernorm",
    "final": "model.norm", "embed": "model.embed_tokens.weight", "lm_head": "lm_head.weight",
}


class StateDictSource:
    """Parameter source for w4a16.models.Decoder backed by a reference-format state dict (see the module docstring)."""

    def __init__(self, cfg: DecoderConfig, state_dict, device):
        self.cfg, self.sd, self.device = cfg, state_dict, torch.device(device)
        self.names = _OPT if cfg.kind == "opt" else _LLAMA

    def _get(self, key, dtype=None):
        if key not in self.sd:
            raise KeyError(f"state dict has no entry '{key}'")
        t = self.sd[key]
        if dtype is not None and t.dtype != dtype:
            raise TypeError(f"'{key}' has dtype {t.dtype}, expected {dtype}")
        return t.to(self.device)

    def linear(self, layer: int, name: str, in_features: int, out_features: int) -> WALinear:
        prefix = self.names["layer"].format(i=layer) + self.names[name]
        g = self.cfg.group_size
        w = self._get(prefix + ".weight", torch.int32)
        zs = self._get(prefix + ".zeros_scales", torch.float16)
        if tuple(w.shape) != (in_features, out_features // 8):
            raise ValueError(f"'{prefix}.weight' has shape {tuple(w.shape)}, expected {(in_features, out_features // 8)} (4-bit, tile-ordered)")
        if tuple(zs.shape) != (in_features // g, 2 * out_features):
            raise ValueError(f"'{prefix}.zeros_scales' has shape {tuple(zs.shape)}, expected {(in_features // g, 2 * out_features)} for group size {g}")
        has_bias = (prefix + ".bias") in self.sd
        lin = WALinear(in_features, out_features, w_bit=4, group_size=g, bias=has_bias, dev=self.device)
        lin.weight, lin.zeros_scales = w.contiguous(), zs.contiguous()
        if has_bias:
            lin.bias = self._get(prefix + ".bias", torch.float16).reshape(1, out_features).contiguous()
        return lin

    def norm(self, layer, name: str, module: nn.Module) -> nn.Module:
        prefix = self.names["final"] if layer is None else self.names["layer"].format(i=layer) + self.names[name]
        with torch.no_grad():
            module.weight.copy_(self._get(prefix + ".weight").to(module.weight.dtype))
            if not isinstance(module, RMSNorm):
                module.bias.copy_(self._get(prefix + ".bias").to(module.bias.dtype))
        return module

    def table(self, name: str, rows: int, cols: int) -> torch.Tensor:
        key = self.names[name]
        if name == "lm_head" and key not in self.sd:           # tied output embedding
            key = self.names["embed"]
        t = self._get(key).to(torch.float16)
        if t.shape[1] != cols or t.shape[0] < rows:
            raise ValueError(f"'{key}' has shape {tuple(t.shape)}, expected at least {(rows, cols)}")
        return t[:rows].contiguous()


def decoder_from_state_dict(cfg: DecoderConfig, state_dict, rank: int = 0, world: int = 1, group=None, device="cuda",
                            exchange=None) -> Decoder:
    """A Decoder (this rank's shard under tensor parallelism) holding the parameters of a reference-format state dict,
    e.g. torch.load("pytorch_model.bin") of a model saved by the reference's opt_infer.py / llama_infer.py."""
    return Decoder(cfg, rank, world, group, device, exchange=exchange, source=StateDictSource(cfg, state_dict, device))
