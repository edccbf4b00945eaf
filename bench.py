#!/usr/bin/env python3
"""Benchmark of the W4A16 hot path on B200.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--no-prefill] [--no-cpu]

Headline (`value`): the OPT-6.7B-shaped decode sweep - M in {1,4,8,16} on (K,N) in
{(4096,4096), (4096,16384), (16384,4096)}, g=128 - as achieved HBM GB/s (algorithmic bytes /
device time), inputs resident in HBM.  One step = the 12 (shape, M) launches, each run once on
every one of SETS distinct weight sets (rotating, so the bytes touched between two uses of a set
exceed the 126 MB L2).  The step is captured in a CUDA graph; K graph replays are timed with CUDA
events on the launching stream.  Extra keys: `e2e` (same sweep through the host-buffer C-ABI call),
`roofline`, `cpu_baseline`, `prefill` (tcgen05 GEMM TFLOP/s, M in {512,2048,8192}), `sweep`
(per-shape decode numbers), `clocks`.

`--impl reference` times the CPU restatement of the reference path (dequantise + fp32 matmul) on
the host cores instead; the reference ships no CPU implementation of its own.
"""
import argparse
import ctypes
import json
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
SETS = 4                                                         # distinct weight sets per shape
WORKLOAD = "OPT-6.7B decode GEMV sweep: M in {1,4,8,16} x (K,N) in {4096x4096, 4096x16384, 16384x4096}, g=128"


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
def cpu_pass(K, N, M, qw_np, zs_np, x):
    import oracle
    w = oracle.dequant_f32(qw_np, zs_np, K, N, G)                 # C + OpenMP, bit-exact dequantisation
    return torch.matmul(x.float(), torch.from_numpy(w).t())       # fp32 matmul on all host threads


class CpuCase:
    """One bounded sample of the workload for the host cores: the K=4096 N=4096 M=16 call."""
    K, N, M = 4096, 4096, 16

    def __init__(self):
        import oracle
        torch.set_num_threads(os.cpu_count() or 1)
        rng = np.random.default_rng(0)
        self.qw = rng.integers(0, 2 ** 32, size=(self.K, self.N // 8), dtype=np.uint32)
        zs = np.empty((self.K // G, 2 * self.N), dtype=np.float16)
        zs[:, 0::2] = rng.integers(5, 11, size=(self.K // G, self.N)) + 64
        zs[:, 1::2] = rng.random((self.K // G, self.N)) * 0.004 + 0.006
        self.zs = zs.view(np.uint16)
        self.x = torch.randn(self.M, self.K).half()
        self.cores = max(oracle.num_threads(), torch.get_num_threads())
        self.bytes = decode_bytes(self.M, self.K, self.N)
        self.run()                                                # warm (library load, thread pools)

    def run(self):
        t0 = time.perf_counter()
        cpu_pass(self.K, self.N, self.M, self.qw, self.zs, self.x)
        return time.perf_counter() - t0


def cpu_baseline(repeat=3):
    case = CpuCase()
    dt = float(np.mean([case.run() for _ in range(repeat)]))
    return dict(value=case.bytes / dt / 1e9, unit=UNIT, cores=case.cores, kind="port",
                sample=f"{repeat} pass(es) of the K=4096 N=4096 M=16 call (dequantise in C/OpenMP + torch fp32 matmul)",
                seconds_per_pass=dt)


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    case = CpuCase()
    for _ in range(args.warmup):
        case.run()
    times = [case.run() for _ in range(args.steps)]
    dt = float(np.sum(times))
    v = case.bytes * args.steps / dt / 1e9
    cb = dict(value=v, unit=UNIT, cores=case.cores, kind="port",
              sample=f"{args.steps} step(s), each one pass of the K=4096 N=4096 M=16 call (dequantise in C/OpenMP + torch fp32 matmul)")
    line = {
        "impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * dt / args.steps, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f16xs4->f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "note": "CPU restatement of the reference path (the reference ships no CPU code for it); "
                                                 "each step is a bounded sample: one K=4096 N=4096 M=16 call"},
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
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-prefill", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--small", action="store_true", help="one weight set, no extras (for profiler captures)")
    ap.add_argument("--graph", choices=["auto", "on", "off"], default="auto",
                    help="capture the step in a CUDA graph (auto: on unless NCCL collectives are in the step)")
    ap.add_argument("--reduce", choices=["fused", "nccl"], default="fused",
                    help="N > 1: how row-parallel outputs are summed - inside the decode kernel through peer memory, or by an NCCL all-reduce")
    ap.add_argument("--verbose", action="store_true", help="progress lines on stderr")
    ap.add_argument("--workload", default="decode-sweep", choices=["decode-sweep", "opt-6.7b", "llama2-7b"],
                    help="decode-sweep (default, the headline metric) or a full random-init W4A16 decoder stack: prefill + greedy decode tokens/s")
    ap.add_argument("--layers", type=int, default=0, help="override the number of decoder layers of a model workload")
    ap.add_argument("--single", default=None, metavar="K,N,M[,ALGO[,REPS]]",
                    help="only launch one shape REPS times over 4 rotating weight sets and exit (driver for ncu captures); "
                         "ALGO 0 auto, 1 skinny, 2 tcgen05")
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
    if args.workload != "decode-sweep":
        run_model(args)
        return

    import quant
    lib = quant.load_library()
    rank = int(os.environ.get("RANK", "0"))

    def note(msg):
        if args.verbose:
            print(f"[bench rank {rank}] {msg}", file=sys.stderr, flush=True)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
        note("process group up")

    sets = 1 if args.small else SETS
    peaks = measured_peaks()
    stream = torch.cuda.Stream(device=dev)
    sp = stream.cuda_stream

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

    weights = {}
    for si, (K, N) in enumerate(DECODE_SHAPES):
        kl, nl, _ = local_shape(K, N)
        weights[(K, N)] = [synth_packed(kl, nl, G, dev, 1234 + 10 * si + s + 100 * rank) for s in range(sets)]
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

    calls = [(M, K, N, s) for s in range(sets) for (K, N) in DECODE_SHAPES for M in DECODE_M]
    step_bytes = sum(decode_bytes(M, K, N) for (M, K, N, s) in calls)
    launches_per_step = len(calls)
    collectives_per_step = sum(1 for (M, K, N, s) in calls if local_shape(K, N)[2])

    # one eager pass (per-device attribute set-up happens here, outside capture), then capture the step
    if dist is not None:
        dist.barrier()                      # ranks enter the first exchange together
    with torch.cuda.stream(stream):
        for c in calls:
            launch(*c, sp)
    stream.synchronize()
    note("eager pass done")

    def check_exchange(where):
        if exchange is not None:
            epoch, err = exchange.status()
            if err:
                raise RuntimeError(f"peer exchange gave up waiting for rank {err - 1} ({where}, after {epoch} calls)")
    check_exchange("eager pass")
    use_graph = args.graph == "on" or (args.graph == "auto" and (world == 1 or exchange is not None))
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
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    with torch.cuda.stream(stream):
        e0.record(stream)
        for _ in range(args.steps):
            run_step()
        e1.record(stream)
    sampler.poll()
    barrier()
    check_exchange("timed region")
    note("timed region done")
    t1 = time.perf_counter()
    clocks = sampler.finish(t0, t1)
    ms = e0.elapsed_time(e1)
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
        "config": {"workload": WORKLOAD, "weight_sets": sets, "launches_per_step": launches_per_step,
                   "l2": f"inputs larger than L2: {sets} rotating weight sets, {step_bytes / 1e6:.0f} MB touched per step",
                   "timing": ("CUDA graph of one step, K replays between CUDA events on the launching stream" if use_graph else
                              "stream-ordered launches (no graph), K steps between CUDA events on the launching stream"),
                   "multi_gpu": (f"tensor parallel over {world} ranks: column-parallel 4096x4096 and 4096x16384, row-parallel "
                                 f"16384x4096 with {collectives_per_step} sums of [M,4096] per step, " +
                                 ("done inside the decode kernel: fp32 partials pushed over NVLink into every rank's exchange buffer, flag hand-shake per CTA"
                                  if exchange is not None else "NCCL fp16 all-reduce after the kernel")) if world > 1 else "single GPU"},
        "gpu_launches": launches_per_step * args.steps,
        "clocks": clocks,
    }
    line["roofline"] = {
        "bound": "hbm", "achieved": per_gpu, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": per_gpu / peaks["hbm_gbs"],
        # dram__bytes_read+write of one ncu capture (K=4096 N=16384 M=1: 35 707 648 B vs 35 692 544 B algorithmic,
        # ratio 1.0004; the other shapes stream their weights the same way), scaled to this mix of launches
        "traffic": 1.0004 * step_bytes / launches_per_step / world, "kernel": "skinny_kernel", "peak_source": f"of {peaks['source']} (copy bandwidth)",
        "algorithmic_bytes_per_launch": step_bytes / launches_per_step / world,
        "avg_launch_us": 1e3 * ms / (args.steps * launches_per_step),
    }

    e2e = None if args.small else e2e_host(lib, weights, dev, stream, sets, world, local_shape)
    if rank == 0 and not args.small:
        if world == 1:
            line["sweep"] = decode_sweep(lib, weights, xs, outs, stream, sets, peaks)
        line["e2e"] = e2e
        if not args.no_prefill and world == 1:
            line["prefill"] = prefill_sweep(lib, weights, dev, stream, sets, peaks)
        if not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline(repeat=5)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(line), flush=True)


def run_model(args):
    """BASELINE configs 4/5: the full decoder stack with every linear W4A16, random init, tensor parallel over
    the ranks torchrun started.  A step = one prompt batch prefilled + greedy decoding; value = decode tokens/s."""
    import torch.distributed as dist
    from w4a16.models import Decoder, DecoderConfig
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    if args.workload == "opt-6.7b":
        cfg, batch, prompt, new = DecoderConfig.opt_6_7b(), 8, 512, 128
    else:
        cfg, batch, prompt, new = DecoderConfig.llama2_7b(), 32, 1024, 256
    if args.layers:
        cfg.layers = args.layers
    exchange = None
    if world > 1 and args.reduce == "fused":
        exchange = make_exchange(32 * cfg.hidden, dev, dist)
    model = Decoder(cfg, rank, world, None, dev, seed=1234, exchange=exchange).mark_static()
    ids = torch.randint(0, cfg.vocab, (batch, prompt), device=dev, generator=torch.Generator(device=dev).manual_seed(7))
    steps, warm = max(1, min(args.steps, 5)), 1
    # NCCL collectives inside graph capture hung on this pool: with --reduce nccl the TP > 1 token steps run eagerly;
    # with the fused exchange the step holds no library collective and is captured at any world size
    graphed = (world == 1 or (exchange is not None and batch <= 32)) and args.graph != "off"
    gen = (lambda n: model.generate_graphed(ids, n, use_graph=True)) if graphed else (lambda n: model.generate_graphed(ids, n, use_graph=False))
    for _ in range(warm):
        gen(8)
    tp, td = [], []
    for _ in range(steps):
        if world > 1:
            dist.barrier()
        _, t_prefill, t_decode = gen(new)
        t = torch.tensor([t_prefill, t_decode], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        tp.append(float(t[0])); td.append(float(t[1]))
        if exchange is not None and exchange.status()[1]:
            raise RuntimeError(f"peer exchange gave up waiting for rank {exchange.status()[1] - 1}")
    prefill_tps = batch * prompt / float(np.mean(tp))
    decode_tps = batch * (new - 1) / float(np.mean(td))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps({
            "metric": f"{args.workload}_w4a16_decode_tokens_per_s", "value": decode_tps, "unit": "tokens/s", "n_gpus": world,
            "steps": steps, "warmup": warm, "ms_per_step": 1e3 * float(np.mean(tp) + np.mean(td)), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f16xs4->f32", "data": "synthetic (random-init packed weights, random token ids)",
            "config": {"workload": args.workload, "layers": cfg.layers, "hidden": cfg.hidden, "ffn": cfg.ffn, "group_size": cfg.group_size,
                       "batch": batch, "prompt_tokens": prompt, "new_tokens": new, "parallelism": f"tp{world}",
                       "attention": "torch scaled_dot_product_attention over a static KV cache (not part of the W4A16 path)",
                       "decode_loop": "one CUDA graph per token step, replayed" if graphed else "eager token steps",
                       "row_parallel_sum": "single GPU" if world == 1 else ("inside the decode kernel through peer memory" if exchange is not None and batch <= 32 else "NCCL fp16 all-reduce"),
                       "timing": "host wall clock around synchronised prefill / decode phases, max over ranks"},
            "prefill_tokens_per_s": prefill_tps, "decode_ms_per_token": 1e3 * float(np.mean(td)) / (new - 1),
        }), flush=True)


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
    for i in range(reps):
        qw, zs = sets[i % 4]
        r = lib.w4a16_gemm_algo(x.data_ptr(), qw.data_ptr(), zs.data_ptr(), None, o.data_ptr(), M, N, K, G, None, 0, None, algo)
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
    with torch.cuda.stream(stream):
        for i in range(warm):
            fn(i)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for i in range(iters):
            fn(i)
        e1.record(stream)
    stream.synchronize()
    return e0.elapsed_time(e1) / iters      # ms per call


def time_graph(fn, stream, launches, replays):
    """ms per launch of `launches` calls captured in one CUDA graph (no host launch cost), rotating weight sets."""
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
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(replays):
            g.replay()
        e1.record(stream)
    stream.synchronize()
    return e0.elapsed_time(e1) / (replays * launches)


def decode_sweep(lib, weights, xs, outs, stream, sets, peaks):
    """Per (shape, M): back-to-back launches inside a CUDA graph, rotating over the weight sets."""
    rows = []
    sp = stream.cuda_stream
    for (K, N) in DECODE_SHAPES:
        for M in DECODE_M:
            def fn(i, sp=sp, M=M, K=K, N=N):
                qw, zs = weights[(K, N)][i % sets]
                lib.w4a16_gemm_ex(xs[(M, K, N)].data_ptr(), qw.data_ptr(), zs.data_ptr(), None, outs[(M, K, N)].data_ptr(),
                                  M, N, K, G, None, 0, sp, 0, 1)
            ms = time_graph(fn, stream, 5 * sets, 10)
            gbs = decode_bytes(M, K, N) / (ms * 1e-3) / 1e9
            rows.append({"K": K, "N": N, "M": M, "us": 1e3 * ms, "GBps": gbs, "frac": gbs / peaks["hbm_gbs"]})
    return rows


def e2e_host(lib, weights, dev, stream, sets, world, local_shape):
    """The same sweep through w4a16_gemm_host: x from pinned host memory, y back to pinned host memory,
    both copies inside the timed region; the packed weights stay resident (module state).  With several
    ranks every rank runs its shard through the host-buffer call (rank 0 reports; no collective here)."""
    sp = stream.cuda_stream
    xh, oh, xd, od = {}, {}, {}, {}
    for (K, N) in DECODE_SHAPES:
        kl, nl, _ = local_shape(K, N)
        for M in DECODE_M:
            xh[(M, K, N)] = torch.randn(M, kl).half().pin_memory()
            oh[(M, K, N)] = torch.empty(M, nl, dtype=torch.float16).pin_memory()
            xd[(M, K, N)] = torch.empty(M, kl, dtype=torch.float16, device=dev)
            od[(M, K, N)] = torch.empty(M, nl, dtype=torch.float16, device=dev)
    calls = [(M, K, N, s) for s in range(sets) for (K, N) in DECODE_SHAPES for M in DECODE_M]

    n_lanes = int(os.environ.get("W4A16_E2E_STREAMS", "4"))
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
    # (b) the step as a batch: every call's copy-in, GEMM and copy-out enqueued with w4a16_gemm_host_async on two
    # streams, ONE synchronisation per step before the results are read
    for c in calls:
        one(c, lib.w4a16_gemm_host_async, lanes[lane_of[c[:3]]])
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        for c in calls:
            one(c, lib.w4a16_gemm_host_async, lanes[lane_of[c[:3]]])
        stream.synchronize()
        for s_ in sides:
            s_.synchronize()
    wall = time.perf_counter() - t0
    return {"value": step_bytes * steps / wall / 1e9, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
            "steps": steps, "ms_per_step": 1e3 * wall / steps,
            "timer": f"host wall clock; per step: all calls enqueued through w4a16_gemm_host_async (pinned host x in, y out) on {len(lanes)} streams, one synchronisation",
            "per_call_sync": {"value": step_bytes * steps / wall_sync / 1e9, "ms_per_step": 1e3 * wall_sync / steps,
                              "device_event_ms_per_step": dev_ms,
                              "what": "w4a16_gemm_host: every call synchronises before it returns"}}


def prefill_sweep(lib, weights, dev, stream, sets, peaks):
    """tcgen05 GEMM: TFLOP/s = 2*M*N*K / time for M in {512, 2048, 8192} on the three shapes."""
    rows = []
    sp = stream.cuda_stream
    for (K, N) in DECODE_SHAPES:
        for M in PREFILL_M:
            x = torch.randn(M, K, device=dev, dtype=torch.float16)
            o = torch.empty(M, N, device=dev, dtype=torch.float16)
            ws_bytes = lib.w4a16_workspace_bytes(M, N, K, G)          # > 0 when the library wants to split K
            ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=dev)

            def fn(i, M=M, K=K, N=N, x=x, o=o, ws=ws, ws_bytes=ws_bytes):
                qw, zs = weights[(K, N)][i % sets]
                r = lib.w4a16_gemm(x.data_ptr(), qw.data_ptr(), zs.data_ptr(), None, o.data_ptr(), M, N, K, G,
                                   ws.data_ptr() if ws_bytes else None, ws_bytes, sp)
                if r != 0:
                    raise RuntimeError(lib.w4a16_status_str(r).decode())
            ms = time_calls(fn, stream, 20, warm=3)
            tf = 2.0 * M * N * K / (ms * 1e-3) / 1e12
            rows.append({"K": K, "N": N, "M": M, "ms": ms, "TFLOPs": tf, "frac_of_measured_bf16_burst": tf / peaks["bf16_tflops"],
                         "frac_of_nominal_2250": tf / 2250.0, "workspace_bytes": ws_bytes})
            del x, o, ws
    flag = ctypes.c_int(0)
    lib.w4a16_device_error_flag(ctypes.byref(flag))
    return {"rows": rows, "kernel": "tc_kernel (TMA + tcgen05.mma, A from TMEM)", "timeout_flag": flag.value,
            "peak_tflops_measured_bf16_burst": peaks["bf16_tflops"]}


if __name__ == "__main__":
    main()
