"""Tensor-parallel sharding of W4A16 linears over one NVLink box (one process per GPU).

The reference has no tensor parallelism (its multi-GPU mode is accelerate's layer placement,
test/nvidia/utils/utils.py:144); this module adds the Megatron-style split the packed format allows
WITHOUT re-quantising:

  column-parallel (q/k/v, fc1, gate/up): split the out-features at multiples of 32.  The `weight`
      buffer is physically [K/32][N/32][32 lanes][4 words] (128 int32 per 32x32 tile), so a shard is
      the tile columns [n0/32, n1/32); `zeros_scales` [K/g, 2N] is sliced at columns [2*n0, 2*n1);
      `bias` [1, N] at [n0, n1).
  row-parallel (out_proj, fc2, o_proj/down): split the in-features at multiples of lcm(32, g).
      32 nominal rows of the [K, N/8] view are one k-tile row, so a shard is the plain row slice
      weight[k0:k1]; `zeros_scales[k0/g:k1/g]`; the bias is added on rank 0 only (once, before the sum).
      Each rank's partial output [tokens, N] is summed with an fp16 all-reduce (NCCL over NVLink).

Uneven shards are allowed (LLaMA's 11008 = 172 groups of 64 -> 22,22,22,22,21,21,21,21 groups at
8 ranks); column shards of gate/up must then use the same boundaries as the row shards of down.
The slicing functions work on tensors of any device, so the rules are tested on CPU ranks (gloo).
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist
from torch import nn

from .qlinear import WALinear


def shard_ranges(total: int, multiple: int, world: int):
    """Split `total` into `world` contiguous ranges whose boundaries are multiples of `multiple`,
    sizes differing by at most one `multiple`; larger shards first.  -> [(begin, end)] * world."""
    assert total % multiple == 0, (total, multiple)
    units = total // multiple
    base, extra = divmod(units, world)
    out, begin = [], 0
    for r in range(world):
        n = (base + (1 if r < extra else 0)) * multiple
        out.append((begin, begin + n))
        begin += n
    assert begin == total
    return out


def shard_column(weight, zeros_scales, bias, n0: int, n1: int):
    """Out-feature shard [n0, n1) (multiples of 32) of a packed linear -> (weight, zeros_scales, bias)."""
    K, n8 = weight.shape
    N = n8 * 8
    assert n0 % 32 == 0 and n1 % 32 == 0 and 0 <= n0 < n1 <= N and K % 32 == 0
    tiles = weight.reshape(K // 32, N // 32, 128)
    w = tiles[:, n0 // 32:n1 // 32, :].contiguous().reshape(K, (n1 - n0) // 8)
    zs = zeros_scales[:, 2 * n0:2 * n1].contiguous()
    b = None if bias is None else bias.reshape(1, N)[:, n0:n1].contiguous()
    return w, zs, b


def shard_row(weight, zeros_scales, bias, k0: int, k1: int, group_size: int, with_bias: bool):
    """In-feature shard [k0, k1) (multiples of lcm(32, group_size)) -> (weight, zeros_scales, bias|None)."""
    K = weight.shape[0]
    m = math.lcm(32, group_size)
    assert k0 % m == 0 and k1 % m == 0 and 0 <= k0 < k1 <= K
    w = weight[k0:k1].contiguous()
    zs = zeros_scales[k0 // group_size:k1 // group_size].contiguous()
    b = bias.contiguous() if (with_bias and bias is not None) else None
    return w, zs, b


def _from_buffers(w, zs, b, group_size):
    K, N = w.shape[0], w.shape[1] * 8
    lin = WALinear(K, N, w_bit=4, group_size=group_size, bias=b is not None, dev=w.device)
    lin.weight, lin.zeros_scales = w, zs
    if b is not None:
        lin.bias = b
    return lin


def fuse_columns(linears):
    """Several W4A16 linears with the same input (q/k/v; gate/up) -> ONE WALinear whose output is their outputs
    side by side, built in the packed domain without re-quantising: the `weight` buffers are [K/32][N_i/32][128]
    tile grids that concatenate along the tile-column axis, `zeros_scales` [K/g, 2N_i] and `bias` [1, N_i] along
    their columns.  The reference carries the same idea as an unused hook (fuse_w1_w3_s4_k_m8, format.cu:114-120).
    Accepts WALinear or ColumnParallelWALinear (their local shard); all must share K, group size and bias-ness."""
    lins = [l.linear if isinstance(l, ColumnParallelWALinear) else l for l in linears]
    K, g = lins[0].in_features, lins[0].group_size
    assert all(l.in_features == K and l.group_size == g for l in lins), "fused linears must share K and group size"
    assert all((l.bias is None) == (lins[0].bias is None) for l in lins), "either all or none of the fused linears carry a bias"
    w = torch.cat([l.weight.reshape(K // 32, l.out_features // 32, 128) for l in lins], dim=1)
    N = sum(l.out_features for l in lins)
    w = w.reshape(K, N // 8).contiguous()
    zs = torch.cat([l.zeros_scales for l in lins], dim=1).contiguous()
    b = None if lins[0].bias is None else torch.cat([l.bias for l in lins], dim=1).contiguous()
    fused = _from_buffers(w, zs, b, g)
    fused.static_weights = all(l.static_weights for l in lins)
    return fused


def fuse_gate_up(gate, up):
    """The gate and up projections of a SwiGLU block -> ONE WALinear whose 32-wide out-feature tiles alternate
    gate, up, gate, up ...: tile 2j of the fused matrix is tile j of `gate`, tile 2j + 1 is tile j of `up`.  With that
    order a (gate, up) pair of the same hidden unit sits 32 columns apart inside one CTA of the decode kernels, which
    can then apply silu(gate) * up in their epilogue (W4A16_FLAG_SILU_MUL, include/w4a16_b200.h) - what the
    reference's fuse_w1_w3_s4_k_m8 (kernel/gemm_s4_f16/format.cu:114-120) prepares for its ops::SiluActivation.
    Built in the packed domain without re-quantising, like fuse_columns.  `split_gate_up` undoes the order on a
    plain output."""
    a, b = [l.linear if isinstance(l, ColumnParallelWALinear) else l for l in (gate, up)]
    K, g, n = a.in_features, a.group_size, a.out_features
    assert b.in_features == K and b.group_size == g and b.out_features == n, "gate and up must have the same shape"
    assert (a.bias is None) == (b.bias is None)
    t = n // 32
    w = torch.stack([a.weight.reshape(K // 32, t, 128), b.weight.reshape(K // 32, t, 128)], dim=2)     # [K/32][t][2][128]
    w = w.reshape(K, 2 * n // 8).contiguous()
    zs = torch.stack([a.zeros_scales.reshape(K // g, t, 64), b.zeros_scales.reshape(K // g, t, 64)], dim=2)
    zs = zs.reshape(K // g, 4 * n).contiguous()
    bias = None
    if a.bias is not None:
        bias = torch.stack([a.bias.reshape(t, 32), b.bias.reshape(t, 32)], dim=1).reshape(1, 2 * n).contiguous()
    fused = _from_buffers(w, zs, bias, g)
    fused.static_weights = a.static_weights and b.static_weights
    return fused


def split_gate_up(y):
    """[..., 2n] output of a fuse_gate_up linear -> (gate [..., n], up [..., n])."""
    n2 = y.shape[-1]
    v = y.reshape(*y.shape[:-1], n2 // 64, 2, 32)
    return v[..., 0, :].reshape(*y.shape[:-1], n2 // 2), v[..., 1, :].reshape(*y.shape[:-1], n2 // 2)


class ColumnParallelWALinear(nn.Module):
    """y_local = x @ W[n0:n1]^T (+ b[n0:n1]); the output stays sharded (feeds attention heads or the
    elementwise activation of the FFN)."""

    def __init__(self, full: WALinear, rank: int, world: int, ranges=None):
        super().__init__()
        g = full.group_size
        ranges = ranges or shard_ranges(full.out_features, 32, world)
        self.n0, self.n1 = ranges[rank]
        w, zs, b = shard_column(full.weight, full.zeros_scales, full.bias, self.n0, self.n1)
        self.linear = _from_buffers(w, zs, b, g)

    def forward(self, x, relu: bool = False, pre_norm=None):
        extra = {}
        if relu:
            extra["relu"] = True
        if pre_norm is not None:
            extra["pre_norm"] = pre_norm
        return self.linear(x, **extra)


class PeerExchange:
    """The exchange buffers of the decode GEMV fused with its all-reduce: one device buffer per rank, every rank's
    buffer mapped into every process through CUDA IPC (all ranks on one node, GPUs peer-accessible).

    capacity = the largest tokens * N of any call that will use it (tokens <= 32).  One object serves all
    row-parallel linears of a model, as long as every rank issues the same calls in the same order on one stream.
    Collective constructor: every rank of `group` must call it.  world == 1 (or no process group) gives a
    single-rank exchange, useful for exercising the kernel path on one GPU.
    """

    def __init__(self, capacity: int, group=None, device=None):
        import ctypes

        import quant
        self.lib = quant.load_library()
        distributed = dist.is_available() and dist.is_initialized()
        self.world = dist.get_world_size(group) if distributed else 1
        self.rank = dist.get_rank(group) if distributed else 0
        self.capacity = int(capacity)
        self.device = torch.device(device if device is not None else torch.cuda.current_device())
        self.buffers = (ctypes.c_void_p * 8)()
        self._opened = []
        self._own = None
        with torch.cuda.device(self.device):
            # Every rank walks through all collective steps whatever happens locally, and the ranks agree on the
            # outcome at the end (which is also the barrier before anyone's first call): a rank that cannot allocate
            # or map must not leave its peers waiting in a collective.
            err = None
            handle = (ctypes.c_ubyte * 64)()
            try:
                own = ctypes.c_void_p()
                quant._check(self.lib.w4a16_exchange_alloc(self.world, self.capacity, ctypes.byref(own)), "exchange_alloc")
                self._own = own
                self.buffers[self.rank] = own.value
                if self.world > 1:
                    quant._check(self.lib.w4a16_exchange_export(own, handle), "exchange_export")
            except Exception as e:                                   # noqa: BLE001
                err = e
            if self.world > 1:
                handles = [None] * self.world
                dist.all_gather_object(handles, bytes(handle), group=group)
                if err is None:
                    try:
                        for r, h in enumerate(handles):
                            if r == self.rank:
                                continue
                            peer = ctypes.c_void_p()
                            raw = (ctypes.c_ubyte * 64).from_buffer_copy(h)
                            quant._check(self.lib.w4a16_exchange_open(raw, ctypes.byref(peer)), "exchange_open")
                            self._opened.append(peer)
                            self.buffers[r] = peer.value
                    except Exception as e:                           # noqa: BLE001
                        err = e
                ok = torch.tensor([0 if err is not None else 1], device=self.device)
                dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
                if int(ok.item()) == 0:
                    self.close()
                    raise RuntimeError(f"peer exchange set-up failed on at least one rank (this rank: {err})")
            elif err is not None:
                raise err

    def allgather(self, t: torch.Tensor) -> torch.Tensor:
        """t: contiguous CUDA tensor of a 4-byte dtype with at most `capacity` elements, same shape on every rank
        -> [world, *t.shape], identical on every rank.  Runs on the current stream; capturable."""
        import quant
        assert t.is_cuda and t.is_contiguous() and t.element_size() == 4 and 0 < t.numel() <= self.capacity
        out = torch.empty((self.world,) + tuple(t.shape), dtype=t.dtype, device=t.device)
        with torch.cuda.device(t.device):
            quant._check(self.lib.w4a16_exchange_allgather(t.data_ptr(), out.data_ptr(), t.numel(), self.buffers, self.world,
                                                           self.rank, self.capacity,
                                                           torch.cuda.current_stream(t.device).cuda_stream), "exchange_allgather")
        return out

    def status(self):
        """-> (calls completed on this rank, error field: 0 or 1 + rank of the peer a wait gave up on)."""
        import ctypes

        import quant
        epoch, err = ctypes.c_uint(0), ctypes.c_int(0)
        with torch.cuda.device(self.device):
            quant._check(self.lib.w4a16_exchange_status(self._own, ctypes.byref(epoch), ctypes.byref(err)), "exchange_status")
        return epoch.value, err.value

    def close(self):
        with torch.cuda.device(self.device):
            for p in self._opened:
                self.lib.w4a16_exchange_close(p)
            self._opened = []
            if self._own is not None:
                self.lib.w4a16_exchange_free(self._own)
                self._own = None


class RowParallelWALinear(nn.Module):
    """y = sum over ranks of x[:, k0:k1] @ W[:, k0:k1]^T + b.

    Two routes to the sum: `exchange` given and at most 32 tokens -> the decode kernel adds the ranks' fp32
    partial sums itself through peer memory (bias added once after the sum); otherwise the local product is
    rounded to fp16 (bias on rank 0) and summed by an fp16 all-reduce over `group`."""

    def __init__(self, full: WALinear, rank: int, world: int, group=None, ranges=None, exchange=None):
        super().__init__()
        g = full.group_size
        ranges = ranges or shard_ranges(full.in_features, math.lcm(32, g), world)
        self.k0, self.k1 = ranges[rank]
        self.k_config = max(k1 - k0 for k0, k1 in ranges)
        w, zs, b = shard_row(full.weight, full.zeros_scales, full.bias, self.k0, self.k1, g, with_bias=(rank == 0))
        self.linear = _from_buffers(w, zs, b, g)
        self.register_buffer("full_bias", None if full.bias is None else full.bias.detach().clone())
        self.group = group
        self.world = world
        self.rank = rank
        self.exchange = exchange
        self._fused_cache = {}

    def _fused_ok(self, tokens: int) -> bool:
        """Whether the fused exchange takes this many tokens for this shard (asked once per token count; the answer
        depends only on shapes, so every rank decides alike)."""
        ok = self._fused_cache.get(tokens)
        if ok is None:
            import quant
            lin = self.linear
            ok = bool(quant.load_library().w4a16_allreduce_supported(tokens, lin.out_features, lin.in_features, self.k_config,
                                                                     lin.group_size, self.exchange.world))
            self._fused_cache[tokens] = ok
        return ok

    def forward(self, x_local, residual=None, stats_out=None):
        """`residual` (the same on all ranks) is added once to the summed output; stats_out: a quant.row_stats_buffer
        that receives the row statistics of the output (up to 16 tokens, decode kernels only)."""
        tokens = x_local.numel() // x_local.shape[-1]
        if self.exchange is not None and tokens <= 32 and tokens * self.linear.out_features <= self.exchange.capacity \
                and self._fused_ok(tokens):
            from quant import gemm_awq_allreduce
            lin = self.linear
            x3 = x_local.reshape(1, tokens, x_local.shape[-1])
            if not x3.is_contiguous():
                x3 = x3.contiguous()
            y = gemm_awq_allreduce(x3, lin.weight, lin.zeros_scales, self.full_bias, lin.out_features, lin.group_size,
                                   self.k_config, self.exchange.buffers, self.exchange.world, self.exchange.rank,
                                   self.exchange.capacity, static_weights=lin.static_weights,
                                   residual=None if residual is None else residual.reshape(1, tokens, lin.out_features).contiguous(),
                                   stats_out=stats_out)
            return y.reshape(*x_local.shape[:-1], lin.out_features)
        if self.world == 1 and residual is not None:
            return self.linear(x_local, residual=residual, stats_out=stats_out)
        y = self.linear(x_local)
        if self.world > 1:
            dist.all_reduce(y, op=dist.ReduceOp.SUM, group=self.group)
        return y if residual is None else y + residual


def mark_static(module: nn.Module, flag: bool = True):
    """Declare the packed buffers of every WALinear below `module` static (see WALinear.static_weights)."""
    for m in module.modules():
        if isinstance(m, WALinear):
            m.static_weights = flag
    return module
