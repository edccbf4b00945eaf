"""One rank of the two-GPU exchange test (started by test_gpu_tp_exchange.py through torch.distributed.run)."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path[:0] = [os.path.dirname(HERE), os.path.join(os.path.dirname(HERE), "sparse-quant_b200"), HERE]

from helpers import check_gemm_tolerance, make_packed, make_x  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    import quant
    from w4a16 import WALinear
    from w4a16.models import Decoder, DecoderConfig
    from w4a16.tp import PeerExchange, RowParallelWALinear, shard_ranges

    ex = PeerExchange(32 * 4096, device=dev)
    # 1. all-gather through the buffers
    mine = torch.arange(24, device=dev, dtype=torch.float32) + 100 * rank
    got = ex.allgather(mine)
    want = torch.stack([torch.arange(24, device=dev, dtype=torch.float32) + 100 * r for r in range(world)])
    assert torch.equal(got, want), "allgather"

    # 2. row-parallel linears: fused sum vs the unsharded product (oracle tolerance), identical on all ranks,
    #    and close to the NCCL route; uneven shards (11 groups of 64 over 2 ranks: 6 + 5)
    for (M, N, K, g) in [(1, 4096, 4096, 128), (8, 1024, 8192, 128), (16, 512, 704, 64), (32, 4096, 2048, 128)]:
        p = make_packed(N, K, g, seed=11 + M)
        full = WALinear(K, N, w_bit=4, group_size=g, bias=True, dev=dev)
        full.weight = torch.from_numpy(p["qweight"].view(np.int32).copy()).to(dev)
        full.zeros_scales = torch.from_numpy(p["zs"].view(np.float16).copy()).to(dev)
        full.bias = (torch.randn(1, N, generator=torch.Generator().manual_seed(5)) * 0.05).half().to(dev)
        ranges = shard_ranges(K, 64 if g == 64 else 128, world)
        fused = RowParallelWALinear(full, rank, world, None, ranges=ranges, exchange=ex)
        nccl = RowParallelWALinear(full, rank, world, None, ranges=ranges)
        x = make_x(M, K, seed=M).to(dev)
        k0, k1 = ranges[rank]
        xl = x[..., k0:k1].contiguous()
        for rep in range(3):
            y = fused(xl)
        y2 = nccl(xl)
        ref = x[0].float().cpu() @ torch.from_numpy(p["w_deq"].astype(np.float32)).t() + full.bias.float().cpu()
        check_gemm_tolerance(y[0], ref, x, p["w_deq"], K)
        check_gemm_tolerance(y2[0], ref, x, p["w_deq"], K)
        every = [torch.empty_like(y) for _ in range(world)]
        dist.all_gather(every, y)
        assert all(torch.equal(every[0], e) for e in every), "fused outputs differ between ranks"
    assert ex.status()[1] == 0

    # 3. a small decoder: the graph-replayed TP step (no library collective inside) against the same step run
    #    eagerly, and logits against the NCCL route
    hidden = max(512, 128 * world)           # every rank's K shard of out_proj must hold whole quantisation groups
    for kind in ("opt", "llama"):
        cfg = (DecoderConfig("opt", layers=2, hidden=hidden, heads=8, ffn=2048, vocab=1024, group_size=128, max_positions=128)
               if kind == "opt" else
               DecoderConfig("llama", layers=2, hidden=hidden, heads=8, ffn=1344, vocab=1024, group_size=64, max_positions=128))
        ids = torch.randint(0, cfg.vocab, (4, 40), device=dev, generator=torch.Generator(device=dev).manual_seed(1))
        model = Decoder(cfg, rank, world, None, dev, seed=5, exchange=ex).mark_static()
        plain = Decoder(cfg, rank, world, None, dev, seed=5).mark_static()
        model.reset(4, 48); plain.reset(4, 48)
        a = model(ids); b = plain(ids)
        tok = b.argmax(-1, keepdim=True)
        a2 = model(tok).float(); b2 = plain(tok).float()       # 4 tokens: fused route vs NCCL route
        rel = ((a2 - b2).norm() / b2.norm()).item()
        assert rel <= 2e-2, rel
        dist.barrier()
        static, _, _ = model.generate_graphed(ids, 6, use_graph=False)
        dist.barrier()
        graphed, _, _ = model.generate_graphed(ids, 6, use_graph=True)
        assert torch.equal(static, graphed), kind
        every = [torch.empty_like(graphed) for _ in range(world)]
        dist.all_gather(every, graphed)
        assert all(torch.equal(every[0], e) for e in every), "ranks decoded different tokens"
    assert ex.status()[1] == 0
    flag = __import__("ctypes").c_int(-1)
    assert quant.load_library().w4a16_device_error_flag(__import__("ctypes").byref(flag)) == 0 and flag.value == 0
    dist.barrier()
    ex.close()
    dist.destroy_process_group()
    if rank == 0:
        print("TP_EXCHANGE_OK", flush=True)


if __name__ == "__main__":
    main()
