"""Tensor-parallel sharding rules of the packed tensors and the row-parallel all-reduce, on CPU ranks
(gloo, world_size 2).  The GPU kernel is replaced by the CPU oracle here (test infrastructure): what is
under test is the host logic - shard boundaries, slicing of the three buffers, bias placement, the
collective, and that a failing rank surfaces as an error on its peer instead of a hang."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from helpers import make_weight


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _packed_linear(N, K, g, seed, bias=True):
    from w4a16 import WALinear
    w = make_weight(N, K, seed)
    qw, zs, _ = oracle.quant_pack(w, g)
    lin = WALinear(K, N, w_bit=4, group_size=g, bias=bias, dev="cpu")
    lin.weight = torch.from_numpy(qw.view(np.int32).copy())
    lin.zeros_scales = torch.from_numpy(zs.view(np.float16).copy())
    if bias:
        gen = torch.Generator().manual_seed(seed + 1)
        lin.bias = (torch.randn(1, N, generator=gen) * 0.05).half()
    return lin


def _oracle_forward(I, W, ZS, bias, N, g, algo=0, out=None, static_weights=False, relu=False):
    """Stand-in for quant.gemm_awq_bias on CPU tensors (same signature)."""
    b, s, K = I.shape
    y = oracle.gemm_awq(I.reshape(-1, K), W.numpy(), ZS.numpy(), N, K, g, None if bias is None else bias.reshape(-1))
    y = torch.from_numpy(y.copy()).reshape(b, s, N)
    return torch.relu(y) if relu else y


def test_shard_ranges_even_and_uneven():
    from w4a16.tp import shard_ranges
    assert shard_ranges(4096, 32, 8) == [(i * 512, (i + 1) * 512) for i in range(8)]
    r = shard_ranges(11008, 64, 8)            # 172 groups of 64 -> 22,22,22,22,21,21,21,21
    assert [b - a for a, b in r] == [1408] * 4 + [1344] * 4
    assert r[0][0] == 0 and r[-1][1] == 11008 and all(r[i][1] == r[i + 1][0] for i in range(7))
    assert all(a % 64 == 0 and a % 32 == 0 for a, _ in r)
    assert [b - a for a, b in shard_ranges(11008, 64, 4)] == [2752] * 4
    with pytest.raises(AssertionError):
        shard_ranges(100, 32, 2)


@pytest.mark.parametrize("N,K,g,world", [(128, 256, 128, 2), (96, 320, 64, 2), (160, 448, 64, 4)])
def test_shards_are_exact_slices_of_the_dequantised_weight(N, K, g, world):
    """No re-quantisation: dequant(shard) is bit-identical to the matching slice of dequant(full)."""
    import math
    from w4a16.tp import shard_column, shard_ranges, shard_row
    lin = _packed_linear(N, K, g, seed=N + K)
    full = oracle.dequant(lin.weight.numpy(), lin.zeros_scales.numpy(), K, N, g)
    for n0, n1 in shard_ranges(N, 32, world):
        w, zs, b = shard_column(lin.weight, lin.zeros_scales, lin.bias, n0, n1)
        assert tuple(w.shape) == (K, (n1 - n0) // 8) and tuple(zs.shape) == (K // g, 2 * (n1 - n0))
        part = oracle.dequant(w.numpy(), zs.numpy(), K, n1 - n0, g)
        assert np.array_equal(part.view(np.uint16), full[n0:n1].view(np.uint16))
        assert torch.equal(b, lin.bias[:, n0:n1])
    for r, (k0, k1) in enumerate(shard_ranges(K, math.lcm(32, g), world)):
        w, zs, b = shard_row(lin.weight, lin.zeros_scales, lin.bias, k0, k1, g, with_bias=(r == 0))
        part = oracle.dequant(w.numpy(), zs.numpy(), k1 - k0, N, g)
        assert np.array_equal(part.view(np.uint16), full[:, k0:k1].view(np.uint16))
        assert (b is not None) == (r == 0)


def _tp_worker(rank, world, port, N, K, g, fail_rank, result):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import datetime
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    try:
        import w4a16.qlinear as ql
        from w4a16.tp import ColumnParallelWALinear, RowParallelWALinear
        ql.gemm_awq_bias = _oracle_forward                       # CPU stand-in for the kernel
        fc1 = _packed_linear(N, K, g, seed=1)                    # column-parallel: K -> N
        fc2 = _packed_linear(K, N, g, seed=2)                    # row-parallel:    N -> K
        gen = torch.Generator().manual_seed(3)
        x = torch.randn(1, 5, K, generator=gen).half()
        ref = ql.WALinear.forward(fc2, torch.relu(ql.WALinear.forward(fc1, x)))
        from w4a16.tp import shard_ranges
        import math
        ranges = shard_ranges(N, math.lcm(32, g), world)          # one set of boundaries for both linears
        c = ColumnParallelWALinear(fc1, rank, world, ranges=ranges)
        r = RowParallelWALinear(fc2, rank, world, ranges=ranges)
        assert (c.n0, c.n1) == (r.k0, r.k1), "column shards of fc1 must match the row shards of fc2"
        h = torch.relu(c(x))
        if rank == fail_rank:
            raise RuntimeError("injected failure before the collective")
        y = r(h)
        err = (y.float() - ref.float()).abs().max().item()
        scale = ref.float().abs().max().item()
        result[rank] = ("ok", err, scale)
    except Exception as e:                                       # noqa: BLE001
        result[rank] = ("error", repr(e)[:200], 0.0)
    finally:
        try:
            dist.destroy_process_group()
        except Exception:                                        # noqa: BLE001
            pass


def _run_tp(N, K, g, fail_rank=-1, world=2):
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        result = mgr.dict()
        port = _free_port()
        procs = [ctx.Process(target=_tp_worker, args=(r, world, port, N, K, g, fail_rank, result)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(timeout=120)
        for p in procs:
            if p.is_alive():
                p.terminate()
                pytest.fail("a tensor-parallel rank hung")
        return dict(result)


@pytest.mark.parametrize("N,K,g", [(256, 128, 128), (320, 128, 64)])     # 320 = 5 groups of 64 -> 3 + 2
def test_column_then_row_parallel_matches_unsharded(N, K, g):
    res = _run_tp(N, K, g)
    assert set(res) == {0, 1}
    for rank in (0, 1):
        status, err, scale = res[rank]
        assert status == "ok", res[rank]
        assert err <= 4e-3 * max(scale, 1.0), (err, scale)         # fp16 partial sums: reassociation only


def test_failing_rank_surfaces_as_error_on_its_peer():
    res = _run_tp(256, 128, 128, fail_rank=1)
    assert res[1][0] == "error" and "injected failure" in res[1][1]
    assert res[0][0] == "error", "rank 0 must see its collective fail (timeout / peer gone), not hang"


def test_fused_sibling_linears_are_the_concatenation_of_their_dequantised_weights():
    """fuse_columns builds q|k|v (or gate|up) in the packed domain: dequantising the fused buffers must give exactly
    the dequantised siblings stacked along the out-feature axis, bias included."""
    from w4a16.tp import fuse_columns
    K, g = 256, 64
    parts = [_packed_linear(n, K, g, seed=20 + i) for i, n in enumerate((96, 32, 160))]
    fused = fuse_columns(parts)
    assert fused.out_features == 288 and fused.in_features == K and fused.group_size == g
    got = oracle.dequant(fused.weight.numpy().view(np.uint32), fused.zeros_scales.numpy().view(np.uint16), K, 288, g)
    want = np.concatenate([oracle.dequant(p.weight.numpy().view(np.uint32), p.zeros_scales.numpy().view(np.uint16), K, p.out_features, g)
                           for p in parts], axis=0)
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))
    assert torch.equal(fused.bias, torch.cat([p.bias for p in parts], dim=1))
    with pytest.raises(AssertionError):
        fuse_columns([parts[0], _packed_linear(32, 128, g, seed=1)])          # different K


def test_gate_up_fusion_alternates_tiles_of_32_out_features():
    """fuse_gate_up interleaves gate and up at tile granularity in the packed domain: rows 64j..64j+31 of the
    dequantised fused matrix are rows 32j..32j+31 of gate, the next 32 those of up; split_gate_up undoes it."""
    from w4a16.tp import fuse_gate_up, split_gate_up
    K, g, n = 256, 64, 96
    gate, up = _packed_linear(n, K, g, seed=31), _packed_linear(n, K, g, seed=32)
    fused = fuse_gate_up(gate, up)
    assert fused.out_features == 2 * n and fused.in_features == K

    def deq(p):
        return oracle.dequant(p.weight.numpy().view(np.uint32), p.zeros_scales.numpy().view(np.uint16), K, p.out_features, g)
    got = deq(fused).reshape(n // 32, 2, 32, K)
    assert np.array_equal(got[:, 0].reshape(n, K).view(np.uint16), deq(gate).view(np.uint16))
    assert np.array_equal(got[:, 1].reshape(n, K).view(np.uint16), deq(up).view(np.uint16))
    b = fused.bias.reshape(n // 32, 2, 32)
    assert torch.equal(b[:, 0].reshape(1, n), gate.bias) and torch.equal(b[:, 1].reshape(1, n), up.bias)
    y = torch.arange(2 * 2 * n, dtype=torch.float32).reshape(2, 2 * n)
    a, c = split_gate_up(y)
    assert torch.equal(a, y.reshape(2, n // 32, 2, 32)[:, :, 0].reshape(2, n))
    assert torch.equal(c, y.reshape(2, n // 32, 2, 32)[:, :, 1].reshape(2, n))


def test_allreduce_supported_is_host_logic():
    """The predicate the row-parallel layer asks before it takes the fused exchange is pure host arithmetic: it answers
    without a GPU, identically for identical shapes."""
    import quant
    lib = quant.load_library()
    assert lib.w4a16_allreduce_supported(8, 4096, 2048, 2048, 128, 8) == 1
    assert lib.w4a16_allreduce_supported(32, 4096, 1344, 1408, 64, 8) == 1
    assert lib.w4a16_allreduce_supported(33, 4096, 2048, 2048, 128, 8) == 0      # more than one pass
    assert lib.w4a16_allreduce_supported(8, 4096, 2048, 1024, 128, 8) == 0       # k_config below this rank's K
    assert lib.w4a16_allreduce_supported(8, 4100, 2048, 2048, 128, 8) == 0       # N not a multiple of 32
