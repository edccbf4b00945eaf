"""Minimal OPT- and LLaMA-shaped decoder stacks built from WALinear, with tensor parallelism.

Only the *shape* of the reference's models matters to the W4A16 path: which tensors go through a
quantised linear and how they are sharded.  This module therefore states the two architectures in a
few lines of torch (embedding, LayerNorm/RMSNorm, RoPE, softmax attention through
torch.nn.functional.scaled_dot_product_attention, static KV cache, greedy decoding) around the
library's linears; it does not reuse the reference's model files (copies of transformers 4.36
internals that do not import under the installed transformers).  Architecture facts follow
test/nvidia/module/opt/modeling_opt_ours.py:532-628 (pre-LN, ReLU, biases, learned positions with
offset 2, q scaled by head_dim**-0.5 after q_proj, tied fp16 lm_head) and
test/nvidia/module/llama/modeling_llama_ours.py:104-158,249-329 (RMSNorm in fp32, rotate-half RoPE,
SwiGLU, no biases, untied fp16 lm_head).

Tensor parallelism (one process per GPU): q/k/v and fc1 (gate/up) column-parallel with attention
heads split across ranks, out_proj and fc2 (down) row-parallel with one all-reduce each, lm_head
split by vocabulary with an all-gather of the logits.  Parameters come from a "source": synthetic by
default (every rank generates the full packed tensors of a layer from the same seed and keeps its exact
shard), or the state dict of a model quantised and saved by the reference (w4a16/checkpoint.py).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.distributed as dist
import torch.nn.functional as F
from torch import nn

from .qlinear import WALinear
from .tp import ColumnParallelWALinear, RowParallelWALinear, fuse_columns, fuse_gate_up, shard_ranges, split_gate_up


@dataclass
class DecoderConfig:
    kind: str = "opt"                 # "opt" | "llama"
    layers: int = 32
    hidden: int = 4096
    heads: int = 32
    ffn: int = 16384
    vocab: int = 50272
    group_size: int = 128
    max_positions: int = 2048
    rope_theta: float = 10000.0
    rms_eps: float = 1e-6
    # token step: normalisations folded into the GEMVs that consume them and residual adds into the GEMVs that produce
    # the block outputs (5 launches per layer); False keeps them as separate add+norm launches (7 per layer)
    fold_norms: bool = True
    fold_norms_max_batch: int = 4

    @staticmethod
    def opt_6_7b():
        return DecoderConfig("opt", 32, 4096, 32, 16384, 50272, 128, 2048)

    @staticmethod
    def llama2_7b():
        return DecoderConfig("llama", 32, 4096, 32, 11008, 32000, 64, 4096)


def synthetic_walinear(in_features, out_features, group_size, bias, seed, device):
    """A WALinear with random packed contents whose dequantised weights look like a quantised N(0, 0.02)
    matrix (nibbles uniform, zero points 5..10, scales U(0.006, 0.010)); deterministic in `seed`."""
    gen = torch.Generator(device=device).manual_seed(seed)
    K, N, g = in_features, out_features, group_size
    lin = WALinear(K, N, w_bit=4, group_size=g, bias=bias, dev=device)
    lin.weight = torch.randint(-2 ** 31, 2 ** 31 - 1, (K, N // 8), dtype=torch.int32, device=device, generator=gen)
    zeros = torch.randint(5, 11, (K // g, N), device=device, generator=gen).to(torch.float16) + 64.0
    scales = (torch.rand((K // g, N), device=device, generator=gen) * 0.004 + 0.006).to(torch.float16)
    lin.zeros_scales = torch.stack([zeros, scales], dim=-1).reshape(K // g, 2 * N).contiguous()
    if bias:
        lin.bias = (torch.randn((1, N), device=device, generator=gen) * 0.02).to(torch.float16)
    return lin


class SyntheticSource:
    """Where a Decoder gets its parameters from.  This one makes them up (random init, deterministic in `seed`): every
    rank generates the full tensors of a layer from the same seed and keeps its exact shard.  checkpoint.StateDictSource
    serves the tensors of a model quantised and saved by the reference instead."""

    def __init__(self, cfg: "DecoderConfig", seed: int, device):
        self.cfg, self.seed, self.device = cfg, seed, device
        self.gen = torch.Generator(device=device).manual_seed(seed)
        self._slots = {"q_proj": 0, "k_proj": 1, "v_proj": 2, "out_proj": 3, "fc1": 4, "gate_proj": 4, "up_proj": 5,
                       "fc2": 6, "down_proj": 6}

    def linear(self, layer: int, name: str, in_features: int, out_features: int) -> WALinear:
        """The full (unsharded) packed linear `name` of decoder layer `layer`."""
        return synthetic_walinear(in_features, out_features, self.cfg.group_size, self.cfg.kind == "opt",
                                  self.seed + 100 * layer + self._slots[name], self.device)

    def norm(self, layer, name: str, module: nn.Module) -> nn.Module:
        """Fill the normalisation `name` ("ln1", "ln2" of a layer, or "final" with layer None); default init here."""
        return module

    def table(self, name: str, rows: int, cols: int) -> torch.Tensor:
        """fp16 [rows, cols]: "embed", "pos_embed" (OPT) or "lm_head" (LLaMA; OPT ties it to "embed")."""
        return (torch.randn((rows, cols), device=self.device, generator=self.gen) * 0.02).to(torch.float16)


class RMSNorm(nn.Module):
    def __init__(self, dim, eps, device):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim, dtype=torch.float16, device=device), requires_grad=False)
        self.eps = eps

    def forward(self, x):
        v = x.float()
        v = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + self.eps)
        return self.weight * v.to(x.dtype)


class DecoderLayer(nn.Module):
    def __init__(self, cfg: DecoderConfig, idx: int, rank: int, world: int, group, device, source, exchange=None):
        super().__init__()
        self.cfg, self.rank, self.world = cfg, rank, world
        H, g = cfg.hidden, cfg.group_size
        self.head_dim = H // cfg.heads
        assert cfg.heads % world == 0, "attention heads must divide evenly over the ranks"
        self.local_heads = cfg.heads // world
        head_ranges = [(r * self.local_heads * self.head_dim, (r + 1) * self.local_heads * self.head_dim) for r in range(world)]
        ffn_ranges = shard_ranges(cfg.ffn, math.lcm(32, g), world)        # shared by fc1/gate/up (columns) and fc2/down (rows)

        def col(name, n_out, ranges):
            return ColumnParallelWALinear(source.linear(idx, name, H, n_out), rank, world, ranges=ranges)

        # q/k/v (and gate/up below) are sharded one by one, then this rank's shards are fused in the packed domain
        # into one linear: one GEMV launch instead of three, and the layout the decode attention kernel reads
        self.qkv_proj = fuse_columns([col("q_proj", H, head_ranges), col("k_proj", H, head_ranges), col("v_proj", H, head_ranges)])
        self.out_proj = RowParallelWALinear(source.linear(idx, "out_proj", H, H), rank, world, group, ranges=head_ranges, exchange=exchange)
        if cfg.kind == "opt":
            self.fc1 = col("fc1", cfg.ffn, ffn_ranges)
            self.ln1 = source.norm(idx, "ln1", nn.LayerNorm(H, device=device, dtype=torch.float16))
            self.ln2 = source.norm(idx, "ln2", nn.LayerNorm(H, device=device, dtype=torch.float16))
            self.fc2 = RowParallelWALinear(source.linear(idx, "fc2", cfg.ffn, H), rank, world, group, ranges=ffn_ranges, exchange=exchange)
        else:
            # gate and up tiles alternate, so that the decode kernel applies silu(gate) * up in its epilogue
            self.gate_up_proj = fuse_gate_up(col("gate_proj", cfg.ffn, ffn_ranges), col("up_proj", cfg.ffn, ffn_ranges))
            self.ln1 = source.norm(idx, "ln1", RMSNorm(H, cfg.rms_eps, device))
            self.ln2 = source.norm(idx, "ln2", RMSNorm(H, cfg.rms_eps, device))
            self.fc2 = RowParallelWALinear(source.linear(idx, "down_proj", cfg.ffn, H), rank, world, group, ranges=ffn_ranges, exchange=exchange)
        self.k_cache = self.v_cache = None

    def alloc_cache(self, batch, max_len, device):
        shape = (batch, self.local_heads, max_len, self.head_dim)
        self.k_cache = torch.zeros(shape, dtype=torch.float16, device=device)
        self.v_cache = torch.zeros(shape, dtype=torch.float16, device=device)

    def forward(self, x, pos0: int, rope=None):
        B, S, H = x.shape
        h = self.ln1(x)
        q, k, v = self.qkv_proj(h).split(self.local_heads * self.head_dim, dim=-1)
        q = q.view(B, S, self.local_heads, self.head_dim).transpose(1, 2)
        k = k.view(B, S, self.local_heads, self.head_dim).transpose(1, 2)
        v = v.view(B, S, self.local_heads, self.head_dim).transpose(1, 2)
        if rope is not None:
            cos, sin = rope
            q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
        self.k_cache[:, :, pos0:pos0 + S] = k
        self.v_cache[:, :, pos0:pos0 + S] = v
        keys, vals = self.k_cache[:, :, :pos0 + S], self.v_cache[:, :, :pos0 + S]
        # scale = head_dim**-0.5 in both architectures (OPT applies it to q after q_proj, :232)
        a = F.scaled_dot_product_attention(q, keys, vals, is_causal=(S > 1 and pos0 == 0))
        a = a.transpose(1, 2).reshape(B, S, self.local_heads * self.head_dim)
        x = x + self.out_proj(a)
        h = self.ln2(x)
        if self.cfg.kind == "opt":
            f = torch.relu(self.fc1(h.reshape(1, B * S, H)))           # the reference's FFN sees [1, B*S, H] (:599-606)
            x = x + self.fc2(f).reshape(B, S, H)
        else:
            gate, up = split_gate_up(self.gate_up_proj(h))
            x = x + self.fc2(F.silu(gate) * up)
        return x


def _norm_args(norm):
    """(weight, bias, eps, rms) of an nn.LayerNorm or RMSNorm, as quant.add_norm takes them."""
    if isinstance(norm, RMSNorm):
        return norm.weight, None, norm.eps, True
    return norm.weight, norm.bias, norm.eps, False


def _layer_forward_static(self, x, pos_t, rope, stats=None):
    """One-token step with the position held in a device tensor (fixed shapes: capturable in a CUDA graph).
    `x` is the residual stream [B, 1, H].  With cfg.fold_norms and up to 16 sequences a layer is five launches: both
    residual adds run in the epilogue of the GEMV that produces the block's output (after the cross-rank sum under
    tensor parallelism), which also leaves the row statistics of the new residual stream; both normalisations run
    inside the GEMV that consumes them, from those statistics.  `stats` = (buffer holding the statistics of x or None,
    buffer for the attention block's output, buffer for this layer's output).  The fused q/k/v GEMV feeds the decode
    attention kernel, which also appends to the cache and applies the rotary embedding (`rope` = the full (cos, sin)
    tables or None).  Returns the new residual stream."""
    from quant import add_norm, decode_attention, silu_mul
    B, S, H = x.shape
    if stats is None:
        _, h = add_norm(x, None, *_norm_args(self.ln1))
        qkv = self.qkv_proj(h).view(B, -1)
        a = decode_attention(qkv, self.k_cache, self.v_cache, pos_t, self.local_heads, rope=rope).view(B, 1, -1)
        x, h = add_norm(x, self.out_proj(a), *_norm_args(self.ln2))
        if self.cfg.kind == "opt":
            return x + self.fc2(self.fc1(h.reshape(1, B, H), relu=True)).reshape(B, 1, H)
        if B <= 32:
            return x + self.fc2(self.gate_up_proj(h, silu_mul=True))
        gate, up = split_gate_up(self.gate_up_proj(h))
        return x + self.fc2(silu_mul(torch.cat((gate, up), dim=-1)))
    s_in, s_mid, s_out = stats
    qkv = self.qkv_proj(x, pre_norm=(*_norm_args(self.ln1), s_in)).view(B, -1)
    a = decode_attention(qkv, self.k_cache, self.v_cache, pos_t, self.local_heads, rope=rope).view(B, 1, -1)
    x = self.out_proj(a, residual=x, stats_out=s_mid)
    ln2 = (*_norm_args(self.ln2), s_mid)
    if self.cfg.kind == "opt":
        f = self.fc1(x.reshape(1, B, H), relu=True, pre_norm=ln2)
        return self.fc2(f, residual=x.reshape(1, B, H), stats_out=s_out).reshape(B, 1, H)
    return self.fc2(self.gate_up_proj(x, silu_mul=True, pre_norm=ln2), residual=x, stats_out=s_out)   # SwiGLU product in the GEMV epilogue


DecoderLayer.forward_static = _layer_forward_static


def apply_rope(x, cos, sin):
    d = x.shape[-1] // 2
    rot = torch.cat((-x[..., d:], x[..., :d]), dim=-1)
    return x * cos + rot * sin


class Decoder(nn.Module):
    def __init__(self, cfg: DecoderConfig, rank: int = 0, world: int = 1, group=None, device="cuda", seed: int = 1234,
                 exchange=None, source=None):
        """exchange: a tp.PeerExchange (capacity >= 32 * hidden).  With it the one-token step contains no library
        collective: row-parallel sums are done inside the decode kernel and the ranks' best logits are gathered
        through the same buffers, so the step can be captured in a CUDA graph at any world size."""
        super().__init__()
        self.cfg, self.rank, self.world, self.group, self.device = cfg, rank, world, group, torch.device(device)
        self.exchange = exchange
        self._row_stats = None            # two quant.row_stats_buffer for the token step (made on first use)
        if source is None:
            source = SyntheticSource(cfg, seed, device)      # `source`: where the parameters come from (see SyntheticSource)
        H = cfg.hidden
        self.embed = source.table("embed", cfg.vocab, H)
        if cfg.kind == "opt":
            self.pos_embed = source.table("pos_embed", cfg.max_positions + 2, H)
            self.final_norm = source.norm(None, "final", nn.LayerNorm(H, device=device, dtype=torch.float16))
        else:
            self.final_norm = source.norm(None, "final", RMSNorm(H, cfg.rms_eps, device))
            inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, H // cfg.heads, 2, device=device).float() / (H // cfg.heads)))
            t = torch.arange(cfg.max_positions, device=device).float()
            emb = torch.cat((torch.outer(t, inv),) * 2, dim=-1)
            self.rope_cos, self.rope_sin = emb.cos().to(torch.float16), emb.sin().to(torch.float16)
        # fp16 lm_head ("lm_head" is in the reference's quant_ignore list), split by vocabulary over the ranks
        self.vocab_ranges = shard_ranges(cfg.vocab, 1, world) if cfg.vocab % world else \
            [(r * cfg.vocab // world, (r + 1) * cfg.vocab // world) for r in range(world)]
        v0, v1 = self.vocab_ranges[rank]
        head_full = self.embed if cfg.kind == "opt" else source.table("lm_head", cfg.vocab, H)
        self.lm_head = head_full[v0:v1].contiguous()
        self.layers = nn.ModuleList(DecoderLayer(cfg, i, rank, world, group, device, source, exchange) for i in range(cfg.layers))
        self.pos = 0

    def mark_static(self):
        """Call once the weights are in place and the device is synchronised (enables weight prefetch)."""
        torch.cuda.synchronize(self.device) if self.device.type == "cuda" else None
        for m in self.modules():
            if isinstance(m, WALinear):
                m.static_weights = True
        return self

    def reset(self, batch, max_len):
        for layer in self.layers:
            layer.alloc_cache(batch, max_len, self.device)
        self.pos = 0

    @torch.no_grad()
    def forward(self, ids):
        """ids [B, S] -> logits of the last position [B, vocab] (fp16); advances the KV cache by S."""
        B, S = ids.shape
        x = self.embed[ids]
        rope = None
        if self.cfg.kind == "opt":
            x = x + self.pos_embed[self.pos + 2:self.pos + 2 + S]
        else:
            rope = (self.rope_cos[self.pos:self.pos + S], self.rope_sin[self.pos:self.pos + S])
        for layer in self.layers:
            x = layer(x, self.pos, rope)
        self.pos += S
        h = self.final_norm(x[:, -1])
        logits = h @ self.lm_head.t()
        if self.world > 1:
            sizes = [b - a for a, b in self.vocab_ranges]
            parts = [torch.empty((B, n), dtype=logits.dtype, device=logits.device) for n in sizes]
            dist.all_gather(parts, logits.contiguous(), group=self.group)
            logits = torch.cat(parts, dim=-1)
        return logits

    @torch.no_grad()
    def step_static(self, tok, pos_t, arange):
        """tok [B, 1] -> next greedy token [B, 1]; position in the device tensor pos_t [1] (advanced here)."""
        x = self.embed[tok]
        rope = None
        if self.cfg.kind == "opt":
            x = x + self.pos_embed.index_select(0, pos_t + 2)
        else:
            rope = (self.rope_cos, self.rope_sin)
        from quant import add_norm
        x = x.contiguous()
        # measured: a gain up to 4 sequences (3 % on one B200, 8 % on four), none at 8, a loss at 16 - every CTA of the
        # consuming GEMV normalises all rows it stages, so the work grows with the batch while the launch it saves does
        # not, and from 5 sequences on the statistics take the small GEMVs off the two-CTAs-per-SM kernel
        fold = self.cfg.fold_norms and x.shape[0] <= self.cfg.fold_norms_max_batch and self.cfg.hidden <= 8192
        if fold and self._row_stats is None:
            from quant import row_stats_buffer
            self._row_stats = tuple(row_stats_buffer(self.cfg.hidden, x.device) for _ in range(2))
        have = False                                     # the first layer's input comes from the embedding: no statistics
        for layer in self.layers:
            if fold:
                mid, out = self._row_stats
                x = layer.forward_static(x, pos_t, rope, (out if have else None, mid, out))
                have = True
            else:
                x = layer.forward_static(x, pos_t, rope)
        _, h = add_norm(x, None, *_norm_args(self.final_norm))
        logits = h[:, -1] @ self.lm_head.t()
        if self.world > 1 and self.exchange is not None:
            # each rank's best (logit, vocabulary index) of its shard; ties go to the lowest rank = lowest index
            val, idx = logits.float().max(-1)
            mine = torch.stack((val, (idx + self.vocab_ranges[self.rank][0]).float())).contiguous()     # [2, B] fp32
            every = self.exchange.allgather(mine)                                                        # [world, 2, B]
            best = every[:, 0].argmax(0, keepdim=True)                                                   # [1, B]
            pos_t += 1
            return every[:, 1].gather(0, best).t().long()
        if self.world > 1:
            parts = [torch.empty_like(logits) for _ in range(self.world)]
            dist.all_gather(parts, logits.contiguous(), group=self.group)
            logits = torch.cat(parts, dim=-1)
        pos_t += 1
        return logits.argmax(-1, keepdim=True)

    @torch.no_grad()
    def generate_graphed(self, prompt_ids, new_tokens: int, use_graph: bool = True):
        """Greedy decoding with the per-token step captured once in a CUDA graph and replayed.
        Returns (tokens, prefill seconds, decode seconds)."""
        import time
        B, S = prompt_ids.shape
        if use_graph and self.world > 1 and (self.exchange is None or B > 32):
            # the step would then hold NCCL collectives (row-parallel sums, logit gather): those are never captured
            # here - the token steps run eagerly instead
            use_graph = False
        max_len = S + new_tokens
        self.reset(B, max_len)
        dev = self.device
        torch.cuda.synchronize(dev)
        t0 = time.perf_counter()
        first = self.forward(prompt_ids).argmax(-1, keepdim=True)
        torch.cuda.synchronize(dev)
        t1 = time.perf_counter()
        tok = first.clone()
        pos_t = torch.full((1,), S, dtype=torch.long, device=dev)
        arange = torch.arange(max_len, device=dev)
        out = torch.empty((B, new_tokens), dtype=torch.long, device=dev)
        out[:, 0:1] = first
        if use_graph:
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(side):                      # warm-up outside capture, then restore the state
                self.step_static(tok, pos_t, arange)
            torch.cuda.current_stream(dev).wait_stream(side)
            pos_t.fill_(S)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                nxt = self.step_static(tok, pos_t, arange)
                tok.copy_(nxt)
            torch.cuda.synchronize(dev)
            if self.world > 1:
                dist.barrier(group=self.group)                 # capture takes host time: start the replays together
                torch.cuda.synchronize(dev)
            t1b = time.perf_counter()
            for i in range(1, new_tokens):
                graph.replay()
                out[:, i:i + 1] = tok
        else:
            t1b = time.perf_counter()
            for i in range(1, new_tokens):
                tok = self.step_static(tok, pos_t, arange)
                out[:, i:i + 1] = tok
        torch.cuda.synchronize(dev)
        t2 = time.perf_counter()
        return out, t1 - t0, t2 - t1b

    @torch.no_grad()
    def generate(self, prompt_ids, new_tokens: int):
        """Greedy decoding; returns (tokens [B, new_tokens], prefill seconds, decode seconds)."""
        B, S = prompt_ids.shape
        self.reset(B, S + new_tokens)
        sync = (lambda: torch.cuda.synchronize(self.device)) if self.device.type == "cuda" else (lambda: None)
        import time
        sync()
        t0 = time.perf_counter()
        nxt = self.forward(prompt_ids).argmax(-1, keepdim=True)
        sync()
        t1 = time.perf_counter()
        out = [nxt]
        for _ in range(new_tokens - 1):
            nxt = self.forward(nxt).argmax(-1, keepdim=True)
            out.append(nxt)
        sync()
        t2 = time.perf_counter()
        return torch.cat(out, dim=1), t1 - t0, t2 - t1
