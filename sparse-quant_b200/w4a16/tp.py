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

    def forward(self, x):
        return self.linear(x)


class RowParallelWALinear(nn.Module):
    """y = sum over ranks of x[:, k0:k1] @ W[:, k0:k1]^T (+ b on rank 0), fp16 all-reduce over `group`."""

    def __init__(self, full: WALinear, rank: int, world: int, group=None, ranges=None):
        super().__init__()
        g = full.group_size
        ranges = ranges or shard_ranges(full.in_features, math.lcm(32, g), world)
        self.k0, self.k1 = ranges[rank]
        w, zs, b = shard_row(full.weight, full.zeros_scales, full.bias, self.k0, self.k1, g, with_bias=(rank == 0))
        self.linear = _from_buffers(w, zs, b, g)
        self.group = group
        self.world = world

    def forward(self, x_local):
        y = self.linear(x_local)
        if self.world > 1:
            dist.all_reduce(y, op=dist.ReduceOp.SUM, group=self.group)
        return y


def mark_static(module: nn.Module, flag: bool = True):
    """Declare the packed buffers of every WALinear below `module` static (see WALinear.static_weights)."""
    for m in module.modules():
        if isinstance(m, WALinear):
            m.static_weights = flag
    return module
