#!/usr/bin/env python3
"""Benchmark of the W4A16 hot path on B200.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--no-prefill] [--no-cpu] [--no-models]

Headline (`value`): the OPT-6.7B-shaped decode sweep - M in {1,4,8,16} on (K,N) in
{(4096,4096), (4096,16384), (16384,4096)}, g=128 - as achieved HBM GB/s (algorithmic bytes /
device time), inputs resident in HBM.  One step = ROUNDS passes over the 12 (shape, M) launches,
ordered batch size by batch size as decode steps run them; every launch of a step reads its own weight set, so no packed byte is read twice within a step and
the bytes that pass between two uses of a set (one whole step) are several times the L2 size.  The
step is captured in a CUDA graph; K replays are timed with CUDA events on the launching stream.
Extra keys: `e2e` (same sweep through the host-buffer C-ABI call), `roofline`, `cpu_baseline`,
`sweep` (per-shape decode numbers, min and median), `prefill` (tcgen05 GEMM TFLOP/s, M in
{512,2048,8192}), `ref_kernel` (the reference's own CUDA kernel rebuilt for sm_100a, timed on the
same box where its rows are self-consistent), `model_opt67b` / `model_llama2_7b` (full decoder
stacks: prefill and decode tokens/s at this number of GPUs), `tp_check` (N > 1: the fused
row-parallel sum against the NCCL route and across ranks), `clocks`.

`--impl reference` times the CPU restatement of the reference path (dequantise + fp32 matmul) on
the host cores instead; the reference ships no CPU implementation of its own.
"""
import argparse
import ctypes
import glob
import importlib.util
import json
import math
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.join(ROOT, "sparse-quant_b200")
for _p in (ROOT, PKG):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import numpy as np
import torch

METRIC = "w4a16_decode_gemv_hbm_gbs"
UNIT = "GB/s"
G = 128
DECODE_SHAPES = [(4096, 4096), (4096, 16384), (16384, 4096)]     # (K, N)
DECODE_M = [1, 4, 8, 16]
PREFILL_M = [512, 2048, 8192]
ROUNDS = 32                                                      # passes over the 12 (shape, M) launches per step
WORKLOAD = "OPT-6.7B decode GEMV sweep: M in {1,4,8,16} x (K,N) in {4096x4096, 4096x16384, 16384x4096}, g=128"
# DRAM bytes moved per algorithmic byte, from an ncu capture of the 12 launches of one round in the step's order
# (profiles/decode_sweep_step_order_launches.md: dram__bytes_read.sum + dram__bytes_write.sum over the launches
# divided by their algorithmic bytes; a little below one because activations and outputs stay in L2)
TRAFFIC_RATIO = 0.9974


def decode_bytes(M, K, N, g=G, bias=False):
    """Algorithmic bytes of one call: packed weights + (zero, scale) pairs + x + y (+ bias)."""
    return K * N // 2 + (K // g) * N * 4 + M * K * 2 + M * N * 2 + (2 * N if bias else 0)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return dict(hbm_gbs=float(d["hbm_gbs"]), bf16_tflops=float(d["bf16_tflops"]),
                    bf16_tflops_sustained=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


# ---------------------------------------------------------------------------------------------
# synthetic packed weights (random nibbles / scales with the value distribution of a quantised
# N(0, 0.02) weight: zero points around 7-8, scales ~ 6 sigma / 15), generated on the device
# ---------------------------------------------------------------------------------------------
def synth_packed(K, N, g, device, seed):
    gen = torch.Generator(device=device).manual_seed(seed)
    qw = torch.randint(-2 ** 31, 2 ** 31 - 1, (K, N // 8), dtype=torch.int32, device=device, generator=gen)
    zeros = torch.randint(5, 11, (K // g, N), device=device, generator=gen).to(torch.float16) + 64.0
    scales = (torch.rand((K // g, N), device=device, generator=gen) * 0.004 + 0.006).to(torch.float16)
    zs = torch.stack([zeros, scales], dim=-1).reshape(K // g, 2 * N).contiguous()
    return qw, zs


class ClockSampler:
    """Polls SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index):
        self.samples = []
        self.stop = False
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.max_mhz = None
        self.t = threading.Thread(target=self._run, daemon=True)

    def poll(self):
        """One sample, taken by the caller's thread (the launching thread calls this right after it has enqueued the
        timed work, so that even a region of a few milliseconds has a sample from inside it)."""
        if not self.ok:
            return
        nv = self.nv
        try:
            mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
            try:
                reasons = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
            except Exception:
                reasons = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
            self.samples.append((time.perf_counter(), mhz, reasons))
        except Exception:
            pass

    def _run(self):
        while not self.stop:
            self.poll()
            time.sleep(0.002)

    def start(self):
        if self.ok:
            self.t.start()

    def finish(self, t0, t1):
        self.stop = True
        if not self.ok:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvml unavailable"]}
        self.t.join(timeout=1.0)
        inside = [s for s in self.samples if t0 <= s[0] <= t1]
        use = inside or self.samples[-3:]
        names = {0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown",
                 0x10: "sync_boost", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
                 0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting"}
        bits = 0
        for s in use:
            bits |= s[2]
        bits &= ~0x1 if inside else bits
        reasons = [n for b, n in names.items() if bits & b]
        mhz = sorted(s[1] for s in use)
        return {"sm_mhz": (mhz[len(mhz) // 2] if mhz else None), "sm_max_mhz": self.max_mhz, "reasons": reasons,
                "samples_in_region": len(inside)}


# ---------------------------------------------------------------------------------------------
# reference / CPU arm
# ---------------------------------------------------------------------------------------------
def cpu_pass(K, N, qw_np, zs_np, x):
    import oracle
    w = oracle.dequant_f32(qw_np, zs_np, K, N, G)                 # C + OpenMP, bit-exact dequantisation
    return torch.matmul(x.float(), torch.from_numpy(w).t())       # fp32 matmul on all host threads


class CpuSweep:
    """The decode sweep on the host cores: per (shape, M) one dequantise (C/OpenMP, all threads) + torch fp32 matmul,
    as the reference's CPU-runnable check does it (dequantise, then matmul)."""

    def __init__(self):
        import oracle
        torch.set_num_threads(os.cpu_count() or 1)
        rng = np.random.default_rng(0)
        self.w = {}
        for (K, N) in DECODE_SHAPES:
            qw = rng.integers(0, 2 ** 32, size=(K, N // 8), dtype=np.uint32)
            zs = np.empty((K // G, 2 * N), dtype=np.float16)
            zs[:, 0::2] = rng.integers(5, 11, size=(K // G, N)) + 64
            zs[:, 1::2] = rng.random((K // G, N)) * 0.004 + 0.006
            self.w[(K, N)] = (qw, zs.view(np.uint16))
        self.x = {(M, K): torch.randn(M, K).half() for (K, _) in DECODE_SHAPES for M in DECODE_M}
        self.cores = max(oracle.num_threads(), torch.get_num_threads())
        self.calls = [(M, K, N) for (K, N) in DECODE_SHAPES for M in DECODE_M]
        self.call(16, 4096, 4096)                                  # warm (library load, thread pools)

    def call(self, M, K, N):
        t0 = time.perf_counter()
        cpu_pass(K, N, *self.w[(K, N)], self.x[(M, K)])
        return time.perf_counter() - t0

    def run(self, calls):
        return sum(self.call(*c) for c in calls)

    def pick_sample(self, steps, budget_s=150.0):
        """The largest sample of the sweep that lets `steps` steps finish within the budget: the 12 calls, the three
        M=16 calls, or the single K=4096 N=4096 M=16 call."""
        per_call = {c: self.call(*c) for c in [(16, K, N) for (K, N) in DECODE_SHAPES]}
        est12 = 4.0 * sum(per_call.values())
        if est12 * steps <= budget_s:
            return self.calls, "the 12 (shape, M) calls of the sweep, once"
        if sum(per_call.values()) * steps <= budget_s:
            return [(16, K, N) for (K, N) in DECODE_SHAPES], "the three M=16 calls of the sweep, once"
        return [(16, 4096, 4096)], "one K=4096 N=4096 M=16 call"


def cpu_baseline():
    sweep = CpuSweep()
    rows = []
    total_t, total_b = 0.0, 0
    for (M, K, N) in sweep.calls:
        dt = sweep.call(M, K, N)
        b = decode_bytes(M, K, N)
        rows.append({"K": K, "N": N, "M": M, "seconds": dt, "GBps": b / dt / 1e9})
        total_t += dt
        total_b += b
    return dict(value=total_b / total_t / 1e9, unit=UNIT, cores=sweep.cores, kind="port",
                sample="one pass of the 12 (shape, M) calls of the sweep (dequantise in C/OpenMP + torch fp32 matmul, all host threads)",
                seconds_per_pass=total_t, rows=rows)


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sweep = CpuSweep()
    calls, what = sweep.pick_sample(args.steps + args.warmup)
    for _ in range(args.warmup):
        sweep.run(calls)
    times = [sweep.run(calls) for _ in range(args.steps)]
    dt = float(np.sum(times))
    nbytes = sum(decode_bytes(*c) for c in calls)
    v = nbytes * args.steps / dt / 1e9
    cb = dict(value=v, unit=UNIT, cores=sweep.cores, kind="port",
              sample=f"{args.steps} step(s), each {what} (dequantise in C/OpenMP + torch fp32 matmul, all host threads)")
    line = {
        "impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * dt / args.steps, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f16xs4->f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "note": "CPU restatement of the reference path (the reference ships no CPU code for it); "
                                                 f"each step is a bounded sample of the sweep: {what}"},
        "cpu_baseline": cb,
        "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------
def make_exchange(capacity, dev, dist):
    """Peer-memory exchange buffers for the fused row-parallel sum, or None when they cannot be set up on this box
    (no peer access / IPC between the ranks): the ranks agree on the outcome, and the caller then falls back to the
    NCCL all-reduce with stream-ordered launches."""
    from w4a16.tp import PeerExchange
    ex, ok = None, 1
    try:
        ex = PeerExchange(capacity, device=dev)
    except Exception as e:                                    # noqa: BLE001
        print(f"[bench] peer exchange set-up failed on rank {dist.get_rank()}: {e}", file=sys.stderr, flush=True)
        ok = 0
    flag = torch.tensor([ok], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if int(flag.item()) == 1:
        return ex
    if ex is not None:
        ex.close()
    return None


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--rounds", type=int, default=ROUNDS, help="passes over the 12 (shape, M) launches per step")
    ap.add_argument("--no-prefill", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-models", action="store_true", help="skip the decoder-stack numbers after the sweep")
    ap.add_argument("--no-ref-kernel", action="store_true", help="skip timing the rebuilt reference kernel")
    ap.add_argument("--small", action="store_true", help="the timed sweep only, no extras (for profiler captures)")
    ap.add_argument("--graph", choices=["auto", "on", "off"], default="auto",
                    help="capture the step in a CUDA graph (never when NCCL collectives are in the step)")
    ap.add_argument("--reduce", choices=["fused", "nccl"], default="fused",
                    help="N > 1: how row-parallel outputs are summed - inside the decode kernel through peer memory, or by an NCCL all-reduce")
    ap.add_argument("--verbose", action="store_true", help="progress lines on stderr")
    ap.add_argument("--decode-kernel", type=int, default=0, help="tuning: 0 automatic, 1 / 2 force one of the two decode kernels")
    ap.add_argument("--workload", default="decode-sweep", choices=["decode-sweep", "opt-6.7b", "llama2-7b"],
                    help="decode-sweep (default, the headline metric) or a full random-init W4A16 decoder stack: prefill + greedy decode tokens/s")
    ap.add_argument("--layers", type=int, default=0, help="override the number of decoder layers of a model workload")
    ap.add_argument("--single", default=None, metavar="K,N,M[,ALGO[,REPS]]",
                    help="only launch one shape REPS times over rotating weight sets and exit (driver for ncu captures); "
                         "ALGO 0 auto, 1 decode kernel, 2 tcgen05")
    ap.add_argument("--single-attention", default=None, metavar="B,H,D,L,POS[,REPS]",
                    help="only launch the decode attention kernel REPS times over 4 rotating caches and exit (driver for ncu captures)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    if args.impl == "reference":
        run_reference(args)
        return
    if args.single:
        run_single(args.single)
        return
    if args.single_attention:
        run_single_attention(args.single_attention)
        return

    import quant
    lib = quant.load_library()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    def note(msg):
        if args.verbose:
            print(f"[bench rank {rank}] {msg}", file=sys.stderr, flush=True)

    if args.workload != "decode-sweep":
        line = model_line(args, args.workload, rank, world, dev, dist)
        if dist is not None:
            dist.barrier()
            dist.destroy_process_group()
        if rank == 0:
            print(json.dumps(line), flush=True)
        return

    if args.decode_kernel:
        lib.w4a16_tune_decode(args.decode_kernel, 0, 0, 0)
    peaks = measured_peaks()
    stream = torch.cuda.Stream(device=dev)
    sp = stream.cuda_stream
    rounds = max(1, args.rounds)
    l2_bytes = torch.cuda.get_device_properties(dev).L2_cache_size

    # Tensor-parallel sharding of the sweep at N > 1 (Megatron style, as the model builder does it):
    #   4096 x 4096  (q/k/v-type) and 4096 x 16384 (fc1): column-parallel, each rank owns N / world out-features;
    #   16384 x 4096 (fc2): row-parallel, each rank owns K / world in-features and the [M, 4096] partial outputs
    #   are summed inside the kernel through peer memory (--reduce fused) or by one NCCL fp16 all-reduce per call.
    #   Total work is fixed: strong scaling.
    def local_shape(K, N):
        if world == 1:
            return K, N, False
        if K > N:
            return K // world, N, True            # row-parallel -> all-reduce
        return K, N // world, False               # column-parallel

    exchange = None
    if world > 1 and args.reduce == "fused":
        exchange = make_exchange(max(DECODE_M) * max(N for _, N in DECODE_SHAPES), dev, dist)
        note("peer exchange buffers mapped" if exchange is not None else "peer exchange unavailable: NCCL all-reduce instead")

    # one weight set per launch of the step: rounds * len(DECODE_M) sets per shape
    sets = rounds * len(DECODE_M)
    weights = {}
    for si, (K, N) in enumerate(DECODE_SHAPES):
        kl, nl, _ = local_shape(K, N)
        weights[(K, N)] = [synth_packed(kl, nl, G, dev, 1234 + 1000 * si + s + 100000 * rank) for s in range(sets)]
    xs, outs = {}, {}
    for (K, N) in DECODE_SHAPES:
        kl, nl, _ = local_shape(K, N)
        for M in DECODE_M:
            xs[(M, K, N)] = torch.randn(M, kl, device=dev, dtype=torch.float16)
            outs[(M, K, N)] = torch.empty(M, nl, device=dev, dtype=torch.float16)

    def launch(M, K, N, s, st):
        qw, zs = weights[(K, N)][s]
        kl, nl, reduce = local_shape(K, N)
        # the packed weights are static module state: W4A16_FLAG_STATIC_WEIGHTS lets a launch prefetch them while
        # the previous kernel of the stream drains (x and out still wait for it)
        if reduce and exchange is not None:
            r = lib.w4a16_gemm_allreduce(xs[(M, K, N)].data_ptr(), qw.data_ptr(), zs.data_ptr(), None, outs[(M, K, N)].data_ptr(),
                                         M, nl, kl, G, kl, exchange.buffers, world, rank, exchange.capacity, st, 1)
        else:
            r = lib.w4a16_gemm_ex(xs[(M, K, N)].data_ptr(), qw.data_ptr(), zs.data_ptr(), None, outs[(M, K, N)].data_ptr(),
                                  M, nl, kl, G, None, 0, st, 0, 1)
        if r != 0:
            raise RuntimeError(lib.w4a16_status_str(r).decode())
        if reduce and exchange is None:
            dist.all_reduce(outs[(M, K, N)])

    # order of a step: batch size by batch size (a decode step runs all its linears at ONE batch size), round by
    # round, shape by shape - consecutive launches never share a weight set
    calls = [(M, K, N, rd * len(DECODE_M) + mi) for mi, M in enumerate(DECODE_M) for rd in range(rounds) for (K, N) in DECODE_SHAPES]
    step_bytes = sum(decode_bytes(M, K, N) for (M, K, N, s) in calls)
    distinct_weight_bytes = sum((K * N // 2 + (K // G) * N * 4) for (M, K, N, s) in calls) // world
    launches_per_step = len(calls)
    collectives_per_step = sum(1 for (M, K, N, s) in calls if local_shape(K, N)[2])

    # one eager pass (per-device attribute set-up happens here, outside capture), then capture the step
    if dist is not None:
        dist.barrier()                      # ranks enter the first exchange together
    with torch.cuda.stream(stream):
        for c in calls[:24]:
            launch(*c, sp)
    stream.synchronize()
    note("eager pass done")

    def check_exchange(where):
        if exchange is not None:
            epoch, err = exchange.status()
            if err:
                raise RuntimeError(f"peer exchange gave up waiting for rank {err - 1} ({where}, after {epoch} calls)")
    check_exchange("eager pass")
    # NCCL collectives are never captured in a graph here: with the NCCL route the launches are stream-ordered
    nccl_in_step = world > 1 and exchange is None
    use_graph = args.graph != "off" and not nccl_in_step
    if args.graph == "on" and nccl_in_step:
        print("[bench] --graph on ignored: the step holds NCCL all-reduces, which are not captured", file=sys.stderr, flush=True)
    if use_graph:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for c in calls:
                launch(*c, torch.cuda.current_stream().cuda_stream)
        note("graph captured")

        def run_step():
            graph.replay()
    else:
        def run_step():
            for c in calls:
                launch(*c, sp)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    with torch.cuda.stream(stream):
        for _ in range(args.warmup):
            run_step()
    barrier()
    check_exchange("warm-up")
    note("warm-up done")
    sampler = ClockSampler(local)
    sampler.start()
    events = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    t0 = time.perf_counter()
    with torch.cuda.stream(stream):
        events[0].record(stream)
        for i in range(args.steps):
            run_step()
            events[i + 1].record(stream)
    sampler.poll()
    barrier()
    check_exchange("timed region")
    note("timed region done")
    t1 = time.perf_counter()
    clocks = sampler.finish(t0, t1)
    ms = events[0].elapsed_time(events[-1])
    step_ms = sorted(events[i].elapsed_time(events[i + 1]) for i in range(args.steps))
    if dist is not None:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    total_bytes = step_bytes * args.steps          # the whole (unsharded) sweep, whatever the number of ranks
    value = total_bytes / (ms * 1e-3) / 1e9
    per_gpu = value / world

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f16xs4->f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "rounds_per_step": rounds, "launches_per_step": launches_per_step,
                   "weight_sets_per_shape": sets,
                   "l2": f"inputs larger than L2: every launch of a step reads its own weight set; {distinct_weight_bytes / 1e6:.0f} MB of "
                         f"distinct packed bytes per GPU pass between two uses of a set (L2 = {l2_bytes / 1e6:.0f} MB)",
                   "timing": ("CUDA graph of one step, K replays between CUDA events on the launching stream" if use_graph else
                              "stream-ordered launches (no graph), K steps between CUDA events on the launching stream"),
                   "multi_gpu": (f"tensor parallel over {world} ranks: column-parallel 4096x4096 and 4096x16384, row-parallel "
                                 f"16384x4096 with {collectives_per_step} sums of [M,4096] per step, " +
                                 ("done inside the decode kernel: fp32 partials pushed over NVLink into every rank's exchange buffer"
                                  if exchange is not None else "NCCL fp16 all-reduce after the kernel")) if world > 1 else "single GPU"},
        "gpu_launches": launches_per_step * args.steps,
        "step_ms": {"min": step_ms[0], "median": step_ms[len(step_ms) // 2], "max": step_ms[-1], "rank": rank},
        "clocks": clocks,
    }
    alg = step_bytes / launches_per_step / world
    line["roofline"] = {
        "bound": "hbm", "achieved": per_gpu, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": per_gpu / peaks["hbm_gbs"],
        "traffic": TRAFFIC_RATIO * alg, "traffic_source": "profiles/decode_sweep_step_order_launches.md (ncu, the 12 launches of one round in the step's order)",
        "kernel": "skinny_kernel (gemv_kernel for 5..8 tokens on matrices up to ~9 MB)", "peak_source": f"of {peaks['source']} (copy bandwidth)",
        "algorithmic_bytes_per_launch": alg,
        "avg_launch_us": 1e3 * ms / (args.steps * launches_per_step),
    }

    if world > 1:
        line["tp_check"] = tp_check(lib, dist, exchange, weights, dev, stream, world, rank, local_shape)
    if not args.small:
        e2e_calls = [(M, K, N, rd * len(DECODE_M) + mi) for mi, M in enumerate(DECODE_M) for rd in range(min(4, rounds)) for (K, N) in DECODE_SHAPES]
        e2e = e2e_host(lib, weights, dev, stream, world, local_shape, e2e_calls)
        if rank == 0:
            line["e2e"] = e2e
        if world == 1:
            line["sweep"] = decode_sweep(lib, weights, xs, outs, stream, peaks)
            if not args.no_prefill:
                line["prefill"] = prefill_sweep(lib, weights, dev, stream, peaks)
            if not args.no_ref_kernel:
                line["ref_kernel"] = ref_kernel_rows(lib, weights, dev, line.get("sweep"), line.get("prefill"))
    # the sweep's buffers are not needed any more
    if exchange is not None:
        exchange.close()
        exchange = None
    del weights, xs, outs
    torch.cuda.empty_cache()
    if not args.small and not args.no_models:
        m = model_line(args, "opt-6.7b", rank, world, dev, dist, steps=2)
        line["model_opt67b"] = {k: m[k] for k in ("value", "unit", "prefill_tokens_per_s", "decode_ms_per_token", "config")}
        if world > 1:
            torch.cuda.empty_cache()
            m = model_line(args, "llama2-7b", rank, world, dev, dist, steps=1)
            line["model_llama2_7b"] = {k: m[k] for k in ("value", "unit", "prefill_tokens_per_s", "decode_ms_per_token", "config")}
    if rank == 0 and not args.small and not args.no_cpu:
        line["cpu_baseline"] = cpu_baseline()
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(line), flush=True)


def tp_check(lib, dist, exchange, weights, dev, stream, world, rank, local_shape):
    """Outside the timed region: the row-parallel product summed inside the kernel against the same partial products
    summed by NCCL (GEMM tolerance), and bit-equality of the fused result across the ranks."""
    if exchange is None:
        return "skipped: no peer exchange (NCCL route timed)"
    K, N = 16384, 4096
    kl, nl, _ = local_shape(K, N)
    qw, zs = weights[(K, N)][0]
    sp = stream.cuda_stream
    verdicts = []
    for M in (1, 16):
        x = torch.randn(M, kl, device=dev, dtype=torch.float16, generator=torch.Generator(device=dev).manual_seed(77 + rank))
        fused = torch.empty(M, nl, device=dev, dtype=torch.float16)
        part = torch.empty(M, nl, device=dev, dtype=torch.float16)
        dist.barrier()
        with torch.cuda.stream(stream):
            r = lib.w4a16_gemm_allreduce(x.data_ptr(), qw.data_ptr(), zs.data_ptr(), None, fused.data_ptr(), M, nl, kl, G, kl,
                                         exchange.buffers, world, rank, exchange.capacity, sp, 0)
            r2 = lib.w4a16_gemm_ex(x.data_ptr(), qw.data_ptr(), zs.data_ptr(), None, part.data_ptr(), M, nl, kl, G, None, 0, sp, 0, 0)
        stream.synchronize()
        if r != 0 or r2 != 0:
            return f"launch failed: {r} {r2}"
        total = part.float()
        dist.all_reduce(total)                                    # fp32 sum of the fp16-rounded partial products
        scale = float(total.abs().max().clamp_min(1e-6))
        close = bool(((fused.float() - total).abs().max() / scale) <= 4e-3)
        ref = fused.clone()
        dist.broadcast(ref, src=0)
        same = torch.tensor([int(torch.equal(ref, fused)) & int(close)], device=dev)
        dist.all_reduce(same, op=dist.ReduceOp.MIN)
        verdicts.append(int(same.item()))
    err = exchange.status()[1]
    if err:
        return f"peer exchange gave up waiting for rank {err - 1}"
    return "ok" if all(verdicts) else f"mismatch (M=1: {verdicts[0]}, M=16: {verdicts[1]})"


MODEL_WORKLOADS = {"opt-6.7b": (8, 512, 128), "llama2-7b": (32, 1024, 256)}      # batch, prompt tokens, new tokens


def model_line(args, workload, rank, world, dev, dist, steps=None):
    """BASELINE configs 4/5: the full decoder stack with every linear W4A16, random init, tensor parallel over
    the ranks torchrun started.  A step = one prompt batch prefilled + greedy decoding; value = decode tokens/s
    (method of the reference's speed test: tokens / wall time of each phase, synchronised)."""
    from w4a16.models import Decoder, DecoderConfig
    cfg = DecoderConfig.opt_6_7b() if workload == "opt-6.7b" else DecoderConfig.llama2_7b()
    batch, prompt, new = MODEL_WORKLOADS[workload]
    if args.layers:
        cfg.layers = args.layers
    exchange = None
    if world > 1 and args.reduce == "fused":
        exchange = make_exchange(32 * cfg.hidden, dev, dist)
    model = Decoder(cfg, rank, world, None, dev, seed=1234, exchange=exchange).mark_static()
    ids = torch.randint(0, cfg.vocab, (batch, prompt), device=dev, generator=torch.Generator(device=dev).manual_seed(7))
    steps = max(1, min(args.steps, 5)) if steps is None else steps
    warm = 1
    # NCCL collectives are never captured in a graph: with --reduce nccl the token steps of N > 1 run eagerly; with
    # the fused exchange the step holds no library collective and is captured at any world size
    graphed = (world == 1 or (exchange is not None and batch <= 32)) and args.graph != "off"
    for _ in range(warm):
        model.generate_graphed(ids, 8, use_graph=graphed)
    tp, td = [], []
    for _ in range(steps):
        if world > 1:
            dist.barrier()
        _, t_prefill, t_decode = model.generate_graphed(ids, new, use_graph=graphed)
        t = torch.tensor([t_prefill, t_decode], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        tp.append(float(t[0])); td.append(float(t[1]))
        if exchange is not None and exchange.status()[1]:
            raise RuntimeError(f"peer exchange gave up waiting for rank {exchange.status()[1] - 1}")
    prefill_tps = batch * prompt / float(np.mean(tp))
    decode_tps = batch * (new - 1) / float(np.mean(td))
    fused = exchange is not None and batch <= 32
    if exchange is not None:
        exchange.close()
    del model
    return {
        "metric": f"{workload}_w4a16_decode_tokens_per_s", "value": decode_tps, "unit": "tokens/s", "n_gpus": world,
        "steps": steps, "warmup": warm, "ms_per_step": 1e3 * float(np.mean(tp) + np.mean(td)), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f16xs4->f32", "data": "synthetic (random-init packed weights, random token ids)",
        "config": {"workload": workload, "layers": cfg.layers, "hidden": cfg.hidden, "ffn": cfg.ffn, "group_size": cfg.group_size,
                   "batch": batch, "prompt_tokens": prompt, "new_tokens": new, "parallelism": f"tp{world}",
                   "attention": "decode: the library's decode attention kernel over a static KV cache; prefill: torch scaled_dot_product_attention",
                   "decode_loop": "one CUDA graph per token step, replayed" if graphed else "eager token steps",
                   "row_parallel_sum": "single GPU" if world == 1 else ("inside the decode kernel through peer memory" if fused else "NCCL fp16 all-reduce"),
                   "timing": "host wall clock around synchronised prefill / decode phases, max over ranks"},
        "prefill_tokens_per_s": prefill_tps, "decode_ms_per_token": 1e3 * float(np.mean(td)) / (new - 1),
    }


def run_single(spec):
    """A handful of launches of one problem, for profiler captures (inputs > L2 via rotating weight sets)."""
    import quant
    lib = quant.load_library()
    v = [int(t) for t in spec.split(",")]
    K, N, M = v[0], v[1], v[2]
    algo = v[3] if len(v) > 3 else 0
    reps = v[4] if len(v) > 4 else 6
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    sets = [synth_packed(K, N, G, dev, 100 + s) for s in range(4)]
    x = torch.randn(M, K, device=dev, dtype=torch.float16)
    o = torch.empty(M, N, device=dev, dtype=torch.float16)
    ws_bytes = lib.w4a16_workspace_bytes(M, N, K, G) if algo != 1 else 0
    ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=dev)
    for i in range(reps):
        qw, zs = sets[i % 4]
        r = lib.w4a16_gemm_algo(x.data_ptr(), qw.data_ptr(), zs.data_ptr(), None, o.data_ptr(), M, N, K, G,
                                ws.data_ptr() if ws_bytes else None, ws_bytes, None, algo)
        if r != 0:
            raise RuntimeError(lib.w4a16_status_str(r).decode())
    torch.cuda.synchronize()
    print(json.dumps({"single": spec, "mean_abs_out": float(o.float().abs().mean())}))


def run_single_attention(spec):
    """A handful of launches of the decode attention kernel on one shape, for profiler captures: B,H,D,L,POS[,REPS]
    (the caches of 4 rotating layers are larger than L2 for the model-sized shapes)."""
    import quant
    v = [int(t) for t in spec.split(",")]
    B, H, D, L, pos = v[:5]
    reps = v[5] if len(v) > 5 else 6
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    caches = [(torch.randn(B, H, L, D, device=dev, dtype=torch.float16), torch.randn(B, H, L, D, device=dev, dtype=torch.float16))
              for _ in range(4)]
    qkv = torch.randn(B, 3 * H * D, device=dev, dtype=torch.float16)
    pos_t = torch.tensor([pos], device=dev)
    for i in range(reps):
        kc, vc = caches[i % 4]
        out = quant.decode_attention(qkv, kc, vc, pos_t, H)
    torch.cuda.synchronize()
    print(json.dumps({"single_attention": spec, "mean_abs_out": float(out.float().abs().mean()),
                      "algorithmic_bytes": 2 * B * H * (pos + 1) * D * 2}))


def time_calls(fn, stream, iters, warm=5):
    """(median, min) ms per call over `iters` calls, each between its own pair of CUDA events on `stream`."""
    with torch.cuda.stream(stream):
        for i in range(warm):
            fn(i)
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(iters + 1)]
        ev[0].record(stream)
        for i in range(iters):
            fn(i)
            ev[i + 1].record(stream)
    stream.synchronize()
    t = sorted(ev[i].elapsed_time(ev[i + 1]) for i in range(iters))
    return t[len(t) // 2], t[0]


def time_graph(fn, stream, launches, replays=7):
    """(median, min) ms per launch of `launches` calls captured in one CUDA graph (no host launch cost) over
    `replays` replays, each between its own pair of CUDA events."""
    with torch.cuda.stream(stream):
        fn(0)
    stream.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=stream):
        for i in range(launches):
            fn(i, torch.cuda.current_stream().cuda_stream)
    with torch.cuda.stream(stream):
        for _ in range(3):
            g.replay()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(replays + 1)]
        ev[0].record(stream)
        for i in range(replays):
            g.replay()
            ev[i + 1].record(stream)
    stream.synchronize()
    t = sorted(ev[i].elapsed_time(ev[i + 1]) / launches for i in range(replays))
    return t[len(t) // 2], t[0]


def decode_sweep(lib, weights, xs, outs, stream, peaks):
    """Per (shape, M): back-to-back launches inside a CUDA graph, rotating over all weight sets of the shape
    (2 x L2 or more of distinct bytes between two uses of a set); median and minimum over 7 replays.  `single_us` is
    the latency of one isolated launch (stream idle before and after)."""
    rows = []
    sp = stream.cuda_stream
    for (K, N) in DECODE_SHAPES:
        sets = weights[(K, N)]
        for M in DECODE_M:
            def fn(i, sp=sp, M=M, K=K, N=N, sets=sets):
                qw, zs = sets[i % len(sets)]
                lib.w4a16_gemm_ex(xs[(M, K, N)].data_ptr(), qw.data_ptr(), zs.data_ptr(), None, outs[(M, K, N)].data_ptr(),
                                  M, N, K, G, None, 0, sp, 0, 1)
            med, mn = time_graph(fn, stream, len(sets))
            singles = []
            for i in range(5):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                stream.synchronize()
                with torch.cuda.stream(stream):
                    e0.record(stream)
                    fn(i + 1)
                    e1.record(stream)
                stream.synchronize()
                singles.append(e0.elapsed_time(e1))
            gbs = decode_bytes(M, K, N) / (med * 1e-3) / 1e9
            rows.append({"K": K, "N": N, "M": M, "us": 1e3 * med, "us_min": 1e3 * mn, "GBps": gbs, "frac": gbs / peaks["hbm_gbs"],
                         "single_us": 1e3 * sorted(singles)[len(singles) // 2], "weight_sets": len(sets)})
    return rows


def e2e_host(lib, weights, dev, stream, world, local_shape, calls):
    """The sweep through w4a16_gemm_host: x from pinned host memory, y back to pinned host memory, both copies inside
    the timed region; the packed weights stay resident (module state).  With several ranks every rank runs its shard
    through the host-buffer call (rank 0 reports; no collective here).  One step here = `calls` (4 rounds)."""
    sp = stream.cuda_stream
    xh, oh, xd, od = {}, {}, {}, {}
    for (K, N) in DECODE_SHAPES:
        kl, nl, _ = local_shape(K, N)
        for M in DECODE_M:
            xh[(M, K, N)] = torch.randn(M, kl).half().pin_memory()
            oh[(M, K, N)] = torch.empty(M, nl, dtype=torch.float16).pin_memory()
            xd[(M, K, N)] = torch.empty(M, kl, dtype=torch.float16, device=dev)
            od[(M, K, N)] = torch.empty(M, nl, dtype=torch.float16, device=dev)

    n_lanes = int(os.environ.get("W4A16_E2E_STREAMS", "12"))          # one per distinct (M, K, N) of the sweep
    sides = [torch.cuda.Stream(device=dev) for _ in range(max(1, n_lanes) - 1)]
    lanes = [sp] + [s_.cuda_stream for s_ in sides]
    lane_of = {key: i % len(lanes) for i, key in enumerate(xh)}       # calls sharing staging buffers stay on one stream

    def one(c, fn, st=None):
        M, K, N, s = c
        qw, zs = weights[(K, N)][s]
        kl, nl, _ = local_shape(K, N)
        r = fn(xh[(M, K, N)].data_ptr(), oh[(M, K, N)].data_ptr(), xd[(M, K, N)].data_ptr(),
               od[(M, K, N)].data_ptr(), qw.data_ptr(), zs.data_ptr(), None, M, nl, kl, G, None, 0,
               sp if st is None else st)
        if r != 0:
            raise RuntimeError(lib.w4a16_status_str(r).decode())

    step_bytes = sum(decode_bytes(M, K, N) for (M, K, N, s) in calls)
    h2d = sum(M * local_shape(K, N)[0] * 2 for (M, K, N, s) in calls)
    d2h = sum(M * local_shape(K, N)[1] * 2 for (M, K, N, s) in calls)
    steps = 20
    # (a) one synchronous call per GEMM (copy in, run, copy out, synchronise): the drop-in call as the module makes it
    for c in calls:
        one(c, lib.w4a16_gemm_host)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    e0.record(stream)
    for _ in range(steps):
        for c in calls:
            one(c, lib.w4a16_gemm_host)
    e1.record(stream)
    stream.synchronize()
    wall_sync = time.perf_counter() - t0
    dev_ms = e0.elapsed_time(e1) / steps
    # (b) the step as a batch: every call's copy-in, GEMM and copy-out enqueued with w4a16_gemm_host_async, ONE
    # synchronisation per step before the results are read.  One host thread per stream submits that stream's calls
    # (the C call releases the interpreter lock; the argument lists are built once, outside the timed region): a
    # single submitting thread was the limit here, not the copies or the kernels.
    import threading
    per_lane = [[] for _ in lanes]
    for c in calls:
        M, K, N, s_ = c
        qw, zs = weights[(K, N)][s_]
        kl, nl, _ = local_shape(K, N)
        lane = lane_of[c[:3]]
        per_lane[lane].append((xh[(M, K, N)].data_ptr(), oh[(M, K, N)].data_ptr(), xd[(M, K, N)].data_ptr(),
                               od[(M, K, N)].data_ptr(), qw.data_ptr(), zs.data_ptr(), None, M, nl, kl, G, None, 0, lanes[lane]))
    fn_async = lib.w4a16_gemm_host_async
    failed = []

    def submit(lane):
        for a in per_lane[lane]:
            r = fn_async(*a)
            if r != 0:
                failed.append(r)

    start, done = threading.Barrier(len(lanes)), threading.Barrier(len(lanes))
    n_steps_total = steps + 1                                    # one untimed pass first

    def worker(lane):
        with torch.cuda.device(dev):
            for _ in range(n_steps_total):
                start.wait()
                submit(lane)
                done.wait()

    threads = [threading.Thread(target=worker, args=(i,), daemon=True) for i in range(1, len(lanes))]
    for t in threads:
        t.start()

    def step():
        start.wait()
        submit(0)
        done.wait()
        stream.synchronize()
        for s_ in sides:
            s_.synchronize()

    step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    wall = time.perf_counter() - t0
    for t in threads:
        t.join()
    if failed:
        raise RuntimeError(lib.w4a16_status_str(failed[0]).decode())
    return {"value": step_bytes * steps / wall / 1e9, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
            "steps": steps, "ms_per_step": 1e3 * wall / steps, "launches_per_step": len(calls),
            "timer": f"host wall clock; per step: all calls enqueued through w4a16_gemm_host_async (pinned host x in, y out) on {len(lanes)} streams, one submitting host thread per stream, one synchronisation",
            "per_call_sync": {"value": step_bytes * steps / wall_sync / 1e9, "ms_per_step": 1e3 * wall_sync / steps,
                              "device_event_ms_per_step": dev_ms,
                              "what": "w4a16_gemm_host: every call synchronises before it returns"}}


def prefill_sweep(lib, weights, dev, stream, peaks):
    """tcgen05 GEMM: TFLOP/s = 2*M*N*K / time for M in {512, 2048, 8192} on the three shapes.  Calls of less than
    about 100 us are timed as 16 back-to-back launches in a CUDA graph rotating over the weight sets (median and
    minimum of 7 replays): one eager call at a time leaves the GPU waiting for the host between launches (24 us in a
    graph against 29 us eagerly at M = 512 on 4096 x 4096).  Longer calls: 20 eager calls, each between its own events."""
    rows = []
    sp = stream.cuda_stream
    for (K, N) in DECODE_SHAPES:
        sets = weights[(K, N)]
        for M in PREFILL_M:
            x = torch.randn(M, K, device=dev, dtype=torch.float16)
            o = torch.empty(M, N, device=dev, dtype=torch.float16)
            ws_bytes = lib.w4a16_workspace_bytes(M, N, K, G)          # > 0 when the library wants to split K
            ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=dev)

            def fn(i, st=None, M=M, K=K, N=N, x=x, o=o, ws=ws, ws_bytes=ws_bytes, sets=sets):
                qw, zs = sets[i % len(sets)]
                r = lib.w4a16_gemm(x.data_ptr(), qw.data_ptr(), zs.data_ptr(), None, o.data_ptr(), M, N, K, G,
                                   ws.data_ptr() if ws_bytes else None, ws_bytes, sp if st is None else st)
                if r != 0:
                    raise RuntimeError(lib.w4a16_status_str(r).decode())
            in_graph = 2.0 * M * N * K < 1.2e11                       # below ~100 us at the rates measured here
            med, mn = time_graph(fn, stream, 16) if in_graph else time_calls(fn, stream, 20, warm=3)
            tf = 2.0 * M * N * K / (med * 1e-3) / 1e12
            rows.append({"K": K, "N": N, "M": M, "ms": med, "ms_min": mn, "TFLOPs": tf, "frac_of_measured_bf16_burst": tf / peaks["bf16_tflops"],
                         "frac_of_nominal_2250": tf / 2250.0, "workspace_bytes": ws_bytes,
                         "timed": "16 launches in a CUDA graph" if in_graph else "eager calls between events"})
            del x, o, ws
    flag = ctypes.c_int(0)
    lib.w4a16_device_error_flag(ctypes.byref(flag))
    return {"rows": rows, "kernel": "tc_kernel (TMA + tcgen05.mma, A from TMEM)", "timeout_flag": flag.value,
            "peak_tflops_measured_bf16_burst": peaks["bf16_tflops"]}


def ref_kernel_rows(lib, weights, dev, sweep_rows, prefill):
    """The reference's own CUDA kernel (gemm_s4_f16_nn, g = 128), rebuilt unmodified for sm_100a by oracle/build_ref.py,
    timed on this GPU next to the numbers above: a same-box comparator, outside every timed region of the product.  It
    launches on the legacy default stream and allocates its output per call, so it is timed as the reference runs it:
    stream-ordered calls between CUDA events on that stream, rotating over the same weight sets.  A row is only timed
    when the kernel's output agrees with this library's on every token row (rebuilt for sm_100a it returns wrong rows
    for some tile configurations); otherwise the row says so."""
    so = glob.glob(os.path.join(ROOT, "oracle", "_ref", "quant*.so"))
    if not so:
        return {"unavailable": "reference extension not built (oracle/build_ref.py needs the reference tree)"}
    try:
        spec = importlib.util.spec_from_file_location("quant", so[0])
        refq = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(refq)
    except Exception as e:                                    # noqa: BLE001
        return {"unavailable": f"reference extension does not load: {e}"}
    mine = {}
    for r in (sweep_rows or []):
        mine[(r["K"], r["N"], r["M"])] = r["us"]
    for r in ((prefill or {}).get("rows") or []):
        mine[(r["K"], r["N"], r["M"])] = 1e3 * r["ms"]
    default = torch.cuda.default_stream(dev)
    rows = []
    for (K, N) in DECODE_SHAPES:
        sets = weights[(K, N)]
        for M in (1, 4, 8, 16, 512, 2048):
            x = torch.randn(1, M, K, device=dev, dtype=torch.float16)
            qw, zs = sets[0]
            with torch.cuda.stream(default):
                ref = refq.gemm_awq_ut(x, qw, zs, M, N, K, G)
            torch.cuda.synchronize()
            own = torch.empty(1, M, N, device=dev, dtype=torch.float16)
            ws_bytes = lib.w4a16_workspace_bytes(M, N, K, G)
            ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=dev)
            st = lib.w4a16_gemm(x.data_ptr(), qw.data_ptr(), zs.data_ptr(), None, own.data_ptr(), M, N, K, G,
                                ws.data_ptr() if ws_bytes else None, ws_bytes, None)
            torch.cuda.synchronize()
            bound = 1e-2 * float(x.abs().max()) * math.sqrt(K) * 0.1           # max |w| of the synthetic weights is ~ 0.1
            bad = int(((ref[0].float() - own[0].float()).abs().amax(dim=1) > bound).sum()) if st == 0 else M
            row = {"K": K, "N": N, "M": M}
            if bad:
                row.update({"us": None, "note": f"wrong rows on sm_100a: {bad} of {M} token rows disagree with this library beyond the GEMM tolerance"})
            else:
                reps = 40 if M <= 16 else 10
                with torch.cuda.stream(default):
                    for i in range(3):
                        refq.gemm_awq_ut(x, *sets[i % len(sets)], M, N, K, G)
                    ev = [torch.cuda.Event(enable_timing=True) for _ in range(reps + 1)]
                    ev[0].record(default)
                    for i in range(reps):
                        refq.gemm_awq_ut(x, *sets[i % len(sets)], M, N, K, G)
                        ev[i + 1].record(default)
                torch.cuda.synchronize()
                t = sorted(ev[i].elapsed_time(ev[i + 1]) for i in range(reps))
                us = 1e3 * t[len(t) // 2]
                row.update({"us": us, "us_min": 1e3 * t[0]})
                if M <= 16:
                    row["GBps"] = decode_bytes(M, K, N) / us / 1e3
                else:
                    row["TFLOPs"] = 2.0 * M * N * K / us / 1e6
                if (K, N, M) in mine:
                    row["this_library_us"] = mine[(K, N, M)]
                    row["speedup"] = us / mine[(K, N, M)]
            rows.append(row)
            del x, ref, own, ws
    return {"kernel": "gemm_s4_f16_nn (mma.sync + cp.async, rebuilt unmodified for sm_100a; oracle/_ref)",
            "timing": "stream-ordered calls on the legacy default stream between CUDA events, median; includes the per-call "
                      "torch::empty and tile selection of the reference's host path", "rows": rows}


if __name__ == "__main__":
    main()
