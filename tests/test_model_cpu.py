"""Decoder stacks + tensor parallelism on CPU ranks: the kernel is replaced by the CPU oracle (test
infrastructure); under test is the model/TP host logic - head split, shared FFN shard boundaries,
row-parallel all-reduce, vocabulary-split lm_head with all-gather, KV cache across decode steps."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from test_tp_cpu import _oracle_forward, _free_port


def _tiny(kind):
    from w4a16.models import DecoderConfig
    if kind == "opt":
        return DecoderConfig("opt", layers=2, hidden=256, heads=4, ffn=512, vocab=128, group_size=128, max_positions=64)
    return DecoderConfig("llama", layers=2, hidden=256, heads=4, ffn=320, vocab=128, group_size=64, max_positions=64)


def _worker(rank, world, port, kind, result):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import datetime
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    try:
        import w4a16.qlinear as ql
        from w4a16.models import Decoder
        ql.gemm_awq_bias = _oracle_forward
        torch.manual_seed(0)
        cfg = _tiny(kind)
        ids = torch.randint(0, cfg.vocab, (2, 5), generator=torch.Generator().manual_seed(7))
        single = Decoder(cfg, 0, 1, None, "cpu", seed=11)
        single.reset(2, 8)
        ref1 = single(ids).float()
        ref2 = single(ref1.argmax(-1, keepdim=True)).float()
        tp = Decoder(cfg, rank, world, None, "cpu", seed=11)
        tp.reset(2, 8)
        out1 = tp(ids).float()
        out2 = tp(ref1.argmax(-1, keepdim=True)).float()
        scale = max(ref1.abs().max().item(), ref2.abs().max().item(), 1e-3)
        err = max((out1 - ref1).abs().max().item(), (out2 - ref2).abs().max().item())
        result[rank] = ("ok", err, scale, tuple(out1.shape))
    except Exception as e:                                       # noqa: BLE001
        import traceback
        result[rank] = ("error", traceback.format_exc()[-600:], 0.0, ())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("kind", ["opt", "llama"])
def test_tensor_parallel_decoder_matches_single_rank(kind):
    ctx = mp.get_context("spawn")
    world = 2
    with ctx.Manager() as mgr:
        result = mgr.dict()
        port = _free_port()
        procs = [ctx.Process(target=_worker, args=(r, world, port, kind, result)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(timeout=300)
        for p in procs:
            if p.is_alive():
                p.terminate()
                pytest.fail("a rank hung")
        res = dict(result)
    for r in range(world):
        status, err, scale, shape = res[r]
        assert status == "ok", err
        assert shape == (2, 128)
        assert err <= 2e-2 * scale, (err, scale)      # fp16 partial sums are re-associated by the split
