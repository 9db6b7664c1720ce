#!/usr/bin/env python
"""Benchmark of the fused pseudorandom-weight matmul (forward + dX + dC) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload gemm|sharded|gemv|gpt2mlp]
                    [--gather-output] [--replicate-grads] [--no-graph] [--no-cpu-baseline] [--no-sharded-record]
                    [--exchange peer|nccl] [--profile-case noise|staged|roles|products|gemv|hash|overlap|formr ...]

One step = one forward + backward pass of the layer over one batch of seeded synthetic input.
Default workload ("gemm"): x bf16 [8192 x 4096], virtual W [16384 x 4096], d_c = 1024, seed 42, float32
accumulation -- the single-GPU configuration the headline metric is quoted on.  With N > 1 (launched by
torchrun, one rank per GPU) every rank runs that step on its own tokens and the coefficient gradients
are summed with one NCCL all-reduce per step (data parallel, weak scaling).

`--workload sharded` runs the 65536 x 16384 virtual layer (d_c = 2048, seed 7) with its output rows split
over the ranks (strong scaling; by default y, dX and dC stay sharded, `--gather-output` all-gathers y and
`--replicate-grads` gives every rank the full dX and dC); `--workload gemv` the batch-1 float32 4096 x 4096 layer
(the step replayed as a CUDA graph unless `--no-graph`); `--workload gpt2mlp` the 24 pseudorandom-weight layers of
GPT-2 small's MLPs (768 <-> 3072, d_c = 128), data parallel with one flat all-reduce of their dC.

The default line also carries a `sharded` sub-record: the row-sharded 65536 x 16384 layer measured right after the headline
in the same process on the same N GPUs (value, ms per step, speed-up over one GPU measured in the same run, device time of
each phase, and the figure with y all-gathered), so one `bench.py --gpus N` run per N gives both scaling curves.

`--profile-case X` runs a small, self-terminating case for a profiler instead of the benchmark (see profile_case()).

Prints ONE JSON line (rank 0).  `--impl reference` times the reference's CPU PyTorch path (explicit noise
matrix, W = S @ C, F.linear, autograd) on the host cores instead; it never touches the GPU kernels.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: T, K, N, R, seed, dtype
    "gemm": dict(T=8192, K=4096, N=16384, R=1024, seed=42, dtype="bf16", coef_std=(3 * 0.02 ** 2 / 1024) ** 0.5),
    "sharded": dict(T=4096, K=16384, N=65536, R=2048, seed=7, dtype="bf16", coef_std=(3 * 0.02 ** 2 / 2048) ** 0.5),
    "gemv": dict(T=1, K=4096, N=4096, R=256, seed=42, dtype="f32", coef_std=(3.0 / (256 * 4096)) ** 0.5),
}


def algorithmic_flops(T, K, N, R):
    """Minimum-association count for fwd + dX + dC: factored 2TR(3K+2N) or the W path 6TNK + 6NRK."""
    fact = 2.0 * T * R * (3 * K + 2 * N)
    wpath = 6.0 * T * N * K + 6.0 * N * R * K
    return min(fact, wpath)


def cpu_model():
    """Name of the host CPU the CPU legs ran on (first 'model name' of /proc/cpuinfo)."""
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.lower().startswith("model name"):
                    return line.split(":", 1)[1].strip()
    except OSError:
        pass
    return "unknown"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return dict(hbm=d["hbm_gbs"], tensor=d["bf16_tflops"], tensor_sustained=d["bf16_tflops_sustained"], src="measured")
    return dict(hbm=6650.0, tensor=1590.0, tensor_sustained=1400.0, src="fallback")


def bind_near_gpu(local: int):
    """Pin this process to the CPU cores of the NUMA node the GPU hangs off (multi-GPU runs only), so that the pinned host
    buffers it allocates afterwards are local to the GPU's PCIe root: with eight ranks copying at once the host side is what
    limits the end-to-end step.  Returns the node, or None when the machine exposes no NUMA placement."""
    try:
        p = torch.cuda.get_device_properties(local)
        bus = f"{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{bus}/numa_node") as f:
            node = int(f.read().strip())
        if node < 0:
            return None
        cpus = set()
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            for part in f.read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = os.sched_getaffinity(0) & cpus
        if not allowed:
            return None
        os.sched_setaffinity(0, allowed)
        return node
    except Exception:
        return None


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.lines, self.proc = gpu_index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50",
                                          "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, t0, t1):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.12)
        self.proc.terminate()
        sm, smax, reasons = [], None, set()
        for ts, line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                clk, mx = float(parts[1]), float(parts[2])
            except ValueError:
                continue
            smax = mx
            if t0 - 0.05 <= ts <= t1 + 0.1:
                sm.append(clk)
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
        if not sm:  # region shorter than the sampling period: use everything seen
            for ts, line in self.lines:
                parts = [p.strip() for p in line.split(",")]
                try:
                    sm.append(float(parts[1]))
                except (ValueError, IndexError):
                    pass
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": smax, "reasons": sorted(reasons),
                "samples": len(sm)}


# --------------------------------------------------------------------------------------------------
# reference arm / CPU baseline: explicit S, W = S @ C, F.linear, autograd -- float32 on the host cores
# --------------------------------------------------------------------------------------------------
def cpu_reference_step(cfg, T_sample, state=None):
    """One forward+backward of the reference's PyTorch path on the CPU; returns (seconds, state)."""
    from oracle import oracle as O  # the CPU baseline leg is one of the places allowed to run the oracle
    K, N, R, seed = cfg["K"], cfg["N"], cfg["R"], cfg["seed"]
    if state is None:
        g = torch.Generator().manual_seed(1003)
        x = torch.randn(T_sample, K, generator=g)
        C = (torch.randn(R, K, generator=g) * cfg["coef_std"])
        dy = torch.randn(T_sample, N, generator=g)
        if cfg["dtype"] == "bf16":
            x, C, dy = x.bfloat16().float(), C.bfloat16().float(), dy.bfloat16().float()
        state = (x, C, dy)
    x, C, dy = state
    t0 = time.perf_counter()
    S = torch.from_numpy(O.c_noise_f32(N, R, seed))        # generation is part of the path and is timed
    xr = x.clone().requires_grad_(True)
    Cr = C.clone().requires_grad_(True)
    W = S @ Cr
    y = torch.nn.functional.linear(xr, W)
    y.backward(dy)
    dt = time.perf_counter() - t0
    return dt, state


def pick_cpu_sample(cfg, budget_s):
    """Largest token count (<= the workload's) whose estimated step time fits the budget."""
    T = cfg["T"]
    probe = min(T, 256)
    cpu_reference_step(cfg, probe)                          # warm the thread pool / page in
    t_probe, _ = cpu_reference_step(cfg, probe)
    fixed = t_probe                                         # mostly the token-independent S, W = S@C, dC part
    t2, _ = cpu_reference_step(cfg, min(T, 2 * probe))
    per_tok = max((t2 - t_probe) / max(min(T, 2 * probe) - probe, 1), 1e-7)
    fixed = max(t_probe - per_tok * probe, 0.0)
    T_fit = int((budget_s - fixed) / per_tok) if budget_s > fixed else probe
    T_s = max(probe, min(T, T_fit))
    if T_s < T:
        T_s = max(probe, (T_s // 256) * 256)
    return T_s


def run_reference(args, cfg):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    torch.set_num_threads(os.cpu_count() or 1)
    cores = torch.get_num_threads()
    T_s = pick_cpu_sample(cfg, budget_s=max(120.0 / max(args.steps + args.warmup, 1), 1.0))
    state = None
    for _ in range(args.warmup):
        _, state = cpu_reference_step(cfg, T_s, state)
    times = []
    for _ in range(args.steps):
        dt, state = cpu_reference_step(cfg, T_s, state)
        times.append(dt)
    total = sum(times)
    flops = algorithmic_flops(T_s, cfg["K"], cfg["N"], cfg["R"]) * args.steps
    value = flops / total / 1e12
    sample = f"{T_s} of {cfg['T']} tokens per step, full K/N/d_c; algorithmic FLOPs of the sample / wall time"
    line = {
        "impl": "reference", "metric": metric_name(args.workload), "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        # same `config` as the GPU arm's line for this --gpus value (the two lines are compared key by key); what differs is said
        # in `reference_arm`: this arm never shards
        "config": workload_config(args.workload, cfg, args.gpus, args.replicate_grads, args.gather_output),
        "reference_arm": f"ONE host process on {cores} threads at any --gpus value (the reference's CPU path does not shard): a ratio "
                         "against an N-GPU line compares N GPUs with this one host",
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "cpu": cpu_model(), "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def metric_name(workload):
    return "fused PRNG-matmul fwd+bwd GB/s" if workload == "gemv" else "fused PRNG-matmul fwd+bwd TFLOP/s"


def workload_config(name, cfg, gpus, replicate_grads=False, gather_output=False):
    sharded = (f"output rows split over {gpus} ranks (zero weight traffic); " +
               ("y all-gathered beside the backward products; " if gather_output else "y stays row-sharded; ") + "z all-gather, " +
               ("g reduce-scatter, dX all-gather, dC all-reduce (gradients replicated on every rank)" if replicate_grads else
                "g all-reduce; dX stays token-sharded and dC input-feature-sharded (every gradient element on one rank)"))
    par = {"gemm": f"dp{gpus} (tokens per rank fixed, dC summed over the ranks after the backward)" if gpus > 1 else "single GPU",
           "sharded": sharded if gpus > 1 else "single GPU",
           "gemv": "replicas only"}[name]
    return {"workload": f"{name}: x[{cfg['T']}x{cfg['K']}] {cfg['dtype']}, virtual W[{cfg['N']}x{cfg['K']}], d_c={cfg['R']}, "
                        f"seed={cfg['seed']}, fwd + dX + dC",
            "parallelism": par, "l2": "inputs and outputs exceed the 126 MB L2 (no explicit flush)" if name != "gemv"
            else "L2 flushed between iterations"}


# --------------------------------------------------------------------------------------------------
# the row-sharded 65536 x 16384 layer (strong scaling): used by `--workload sharded` and by the `sharded` sub-record
# --------------------------------------------------------------------------------------------------
class ShardedLayerBench:
    """Inputs and step function of the row-sharded layer on this rank.  `exchange`: "peer" = the library's own kernels over
    peer memory when the ranks can map each other's buffers (else NCCL), "nccl" = NCCL collectives between the products."""

    def __init__(self, cfg, dev, world, rank, rb, K, exchange="peer"):
        import torch.distributed as dist
        self.cfg, self.dev, self.world, self.rank, self.rb, self.K, self.dist = cfg, dev, world, rank, rb, K, dist
        T, Kin, N, R = cfg["T"], cfg["K"], cfg["N"], cfg["R"]
        self.plan = rb.parallel.ShardedLayerPlan(T, N, world, rank)
        self.row0, self.n_local = self.plan.row_lo, self.plan.row_hi - self.plan.row_lo
        g = torch.Generator().manual_seed(1005)
        self.x = torch.randn(T, Kin, generator=g).bfloat16().to(dev)
        self.C = (torch.randn(R, Kin, generator=torch.Generator().manual_seed(7)) * cfg["coef_std"]).bfloat16().to(dev)
        gd = torch.Generator(device=dev).manual_seed(2000 + rank)
        self.dy = torch.randn(T, self.n_local, device=dev, generator=gd).bfloat16()
        self.ex = None
        if world > 1 and exchange == "peer":
            self.ex = rb.parallel.PeerExchange.create(self.plan, R, dev)
        self.exchange = "single GPU" if world == 1 else (f"library kernels over peer memory ({self.ex.how})" if self.ex is not None
                                                         else "NCCL collectives between the products")
        self.y_all = None

    def step(self, gather_output=False, replicate=False, timer=None, keep_noise=False):
        rb, K, plan, seed = self.rb, self.K, self.plan, self.cfg["seed"]
        if self.world == 1:
            y = K.linear_fwd(self.x, self.C, seed, self.n_local, self.row0)
            if timer is not None:
                timer.mark("forward (z, noise fill, y)")
            dx, dc = K.linear_bwd(self.dy, self.x, self.C, seed, self.row0)
            if timer is not None:
                timer.mark("backward (noise fill, g, dX, dC)")
            return y, dx, dc
        if self.ex is not None and not replicate:
            y = rb.parallel.sharded_forward_peer(self.x, self.C, seed, plan, self.ex, timer)
        else:
            y = rb.parallel.sharded_forward(self.x, self.C, seed, plan)
            if timer is not None:
                timer.mark("forward (z, z all-gather, y)")
        work = None
        if gather_output:
            if self.y_all is None:
                self.y_all = torch.empty((self.world * self.cfg["T"], self.n_local), dtype=torch.bfloat16, device=self.dev)
            # every rank receives all column blocks of y (rank-major [G, T, N/G]); runs beside the backward products
            work = self.dist.all_gather_into_tensor(self.y_all, y, async_op=True)
        if self.ex is not None and not replicate:
            dx, dc = rb.parallel.sharded_backward_peer(self.dy, self.x, self.C, seed, plan, self.ex, timer, keep_noise=keep_noise)
        else:
            dx, dc = rb.parallel.sharded_backward(self.dy, self.x, self.C, seed, plan, replicate=replicate)
            if timer is not None:
                timer.mark("backward (g, g exchange, dX, dC)")
        if work is not None:
            work.wait()
            if timer is not None:
                timer.mark("y all-gather tail")
        return y, dx, dc

    def timed(self, steps, warmup, **kw):
        """ms per step, maximum over the ranks (barrier and synchronise on both sides of the timed region)."""
        dist, dev = self.dist, self.dev
        for _ in range(max(warmup, 3)):
            self.step(**kw)
        if self.world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            self.step(**kw)
        e1.record()
        if self.world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        self.K.check_status()
        t = torch.tensor([e0.elapsed_time(e1) / steps], device=dev)
        if self.world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def phases(self, reps=5, **kw):
        """Device time of every phase as this rank's launching stream sees it, averaged over `reps` steps (exchanges that
        run on a side stream show up only as the time the main stream waits for them)."""
        acc = {}
        for _ in range(reps):
            self.step(**kw)                      # keeps the GPU busy while the timed step is being enqueued: its first phase
            timer = self.rb.parallel.PhaseTimer()   # then starts from a running stream, not from an idle device
            self.step(timer=timer, **kw)
            torch.cuda.synchronize()
            for k, v in timer.durations().items():
                acc[k] = acc.get(k, 0.0) + v / reps
        return {k: round(v, 4) for k, v in acc.items()}


def sharded_record(args, dev, world, rank, rb, K):
    """The `sharded` sub-record of the default line (also the body of `--workload sharded`)."""
    cfg = WORKLOADS["sharded"]
    T, Kin, N, R = cfg["T"], cfg["K"], cfg["N"], cfg["R"]
    flops = algorithmic_flops(T, Kin, N, R)
    peaks = measured_peaks()
    b = ShardedLayerBench(cfg, dev, world, rank, rb, K, exchange=args.exchange)
    ms = b.timed(args.steps, args.warmup)
    rec = {"workload": workload_config("sharded", cfg, world)["workload"], "n_gpus": world, "scaling": "strong",
           "unit": "TFLOP/s", "value": flops / (ms * 1e-3) / 1e12, "ms_per_step": ms, "steps": args.steps,
           "exchange": b.exchange, "outputs": "y row-sharded (each rank keeps its columns), dX token-sharded, dC input-feature-sharded",
           "phases_ms": b.phases()}
    rec["frac_of_peak_per_gpu"] = rec["value"] / world / peaks["tensor"]
    if world > 1:
        # the same layer on ONE GPU, measured by every rank at the same time in this same process: the denominator of the speed-up
        one = ShardedLayerBench(cfg, dev, 1, 0, rb, K)
        ms1 = one.timed(args.steps, args.warmup)
        del one
        torch.cuda.empty_cache()
        rec["single_gpu_ms_per_step"] = ms1
        rec["speedup_vs_single_gpu"] = ms1 / ms
        ms_g = b.timed(args.steps, args.warmup, gather_output=True)
        rec["gather_output"] = {"what": "the same step with y all-gathered over NVLink (NCCL, beside the backward products): every rank "
                                        "receives (G-1)/G of 537 MB", "ms_per_step": ms_g, "value": flops / (ms_g * 1e-3) / 1e12,
                                "speedup_vs_single_gpu": ms1 / ms_g}
        if b.ex is not None and args.exchange == "peer":
            nccl = ShardedLayerBench(cfg, dev, world, rank, rb, K, exchange="nccl")
            ms_n = nccl.timed(args.steps, args.warmup)
            rec["nccl_exchange"] = {"what": "the same step with NCCL all-gather / all-reduce between the products", "ms_per_step": ms_n,
                                    "value": flops / (ms_n * 1e-3) / 1e12, "speedup_vs_single_gpu": ms1 / ms_n}
            del nccl
            ms_k = b.timed(args.steps, args.warmup, keep_noise=True)
            rec["keep_noise"] = {"what": "the same step with this rank's noise rows kept from the forward to the backward (hashed once "
                                         "per step instead of twice; the single-GPU step it is compared with still hashes twice, as "
                                         "the stateless entry points do, so this is not the like-for-like figure: `value` is)",
                                 "ms_per_step": ms_k, "value": flops / (ms_k * 1e-3) / 1e12, "speedup_vs_single_gpu": ms1 / ms_k}
    else:
        rec["single_gpu_ms_per_step"], rec["speedup_vs_single_gpu"] = ms, 1.0
    del b
    torch.cuda.empty_cache()
    return rec


# --------------------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------------------
def run_ours(args, cfg):
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py measures the CUDA kernels; no GPU is visible (there is no CPU fallback)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    numa_node = bind_near_gpu(local) if world > 1 else None
    if world > 1:
        # NCCL prints its version banner on stdout at NCCL_DEBUG=VERSION; stdout carries the one JSON line only
        if os.environ.get("NCCL_DEBUG", "VERSION").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"
        dist.init_process_group("nccl", device_id=dev)
    from randumb_b200 import kernels as K
    import randumb_b200 as rb

    dt = torch.bfloat16 if cfg["dtype"] == "bf16" else torch.float32
    T, Kin, N, R, seed = cfg["T"], cfg["K"], cfg["N"], cfg["R"], cfg["seed"]
    row0, n_local = 0, N
    sb = None
    if args.workload == "sharded":
        sb = ShardedLayerBench(cfg, dev, world, rank, rb, K, exchange=args.exchange)
        row0, n_local = sb.row0, sb.n_local
        x, C, dy = sb.x, sb.C, sb.dy
        x_host = x.cpu().pin_memory()
    else:
        g = torch.Generator().manual_seed(1003 + (rank if args.workload == "gemm" else 0))
        x_host = torch.randn(T, Kin, generator=g).to(dt).pin_memory()
        C = (torch.randn(R, Kin, generator=torch.Generator().manual_seed(7)) * cfg["coef_std"]).to(dt).to(dev)
        x = x_host.to(dev)
        dy = torch.randn(T, n_local, generator=g).to(dt).to(dev)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev) if args.workload == "gemv" else None

    # data parallel: the coefficient gradient is summed by the library's kernels over peer memory when the ranks can map each
    # other's buffers (RANDUMB_B200_DP_ALLREDUCE=nccl: always NCCL)
    dc_sum = None
    if world > 1 and sb is None and args.workload != "gemv" and os.environ.get("RANDUMB_B200_DP_ALLREDUCE", "peer") != "nccl":
        dc_sum = rb.parallel.PeerAllReduce.create(R * Kin, dev)

    def step():
        if sb is not None:
            # rows split over ranks: z gathered, g summed; by default dX stays token-sharded and dC input-feature-sharded
            return sb.step(args.gather_output, args.replicate_grads)
        y = K.linear_fwd(x, C, seed, n_local, row0)
        if world > 1:
            # data parallel: the library's backward, then the all-reduce of dC
            dx, dc = rb.parallel.data_parallel_backward(dy, x, C, seed, row0, peer=dc_sum)
        else:
            dx, dc = K.linear_bwd(dy, x, C, seed, row0)
        return y, dx, dc

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
        if flush is not None:
            flush.zero_()
    barrier()
    run, eager_ms = step, None
    if args.workload == "gemv" and not args.no_graph:
        # batch-1 steps are four short kernels: time them eagerly once, then replay them as one CUDA graph so the
        # launch gaps between them are not what is measured
        eager_ms = 0.0
        for _ in range(args.steps):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); step(); e1.record()
            torch.cuda.synchronize()
            eager_ms += e0.elapsed_time(e1)
        eager_ms /= args.steps
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            graph_out = step()
        run = graph.replay
        for _ in range(3):
            run()
        torch.cuda.synchronize()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.15)
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_wall0 = time.time()
    step_ms = None
    if flush is None:
        marks = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]   # one event per step boundary
        ev0.record()
        marks[0].record()
        for i in range(args.steps):
            step()
            marks[i + 1].record()
        ev1.record()
        barrier()
        elapsed_ms = ev0.elapsed_time(ev1)
        step_ms = sorted(marks[i].elapsed_time(marks[i + 1]) for i in range(args.steps))
    else:
        elapsed_ms = 0.0
        for _ in range(args.steps):
            flush.zero_()
            ev0.record()
            run()
            ev1.record()
            torch.cuda.synchronize()
            elapsed_ms += ev0.elapsed_time(ev1)
        barrier()
    t_wall1 = time.time()
    clocks = sampler.stop(t_wall0, t_wall1) if rank == 0 else None
    K.check_status()
    tmax = torch.tensor([elapsed_ms], device=dev)
    if world > 1:
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
    elapsed_ms = float(tmax.item())

    # ---- dominant kernel, timed live with CUDA events on the launching stream -------------------
    roofline, peaks = None, measured_peaks()
    staged = args.workload != "gemv" and K.linear_stages_noise(T, Kin, n_local, R, dt, K.PATH_FACTORED)
    if args.workload != "gemv":
        z = torch.randn(T, R, device=dev).to(dt)
        reps = max(args.steps, 5)

        def time_pair(f_y, f_g):
            evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(2 * reps)]
            for _ in range(2):
                f_y(); f_g()
            torch.cuda.synchronize()
            for i in range(reps):
                evs[2 * i][0].record(); f_y(); evs[2 * i][1].record()
                evs[2 * i + 1][0].record(); f_g(); evs[2 * i + 1][1].record()
            torch.cuda.synchronize()
            return sum(a.elapsed_time(b) for a, b in evs) / len(evs)

        flops_launch = 2.0 * T * n_local * R
        fused_ms = time_pair(lambda: K.gemm_noise(z, n_local, seed, False, row0, impl=K.IMPL_UMMA),
                             lambda: K.gemm_noise(dy, R, seed, True, row0, impl=K.IMPL_UMMA))
        fused = {"kernel": "noise_pair_kernel, two CTA pairs per cluster sharing every generated stage (y = z S^T and g = dY S): S regenerated in shared memory per 512-token tile",
                 "avg_launch_ms": fused_ms, "achieved": flops_launch / (fused_ms * 1e-3) / 1e12}
        if staged:
            S = K.noise(n_local, R, seed, row0, 0, dt, dev)
            avg_ms = time_pair(lambda: K.gemm_dense(z, S), lambda: K.gemm_dense(dy, S, True, False))
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            for _ in range(20):                  # back to back into one buffer, so the interval is device time and not launch overhead
                K.noise(n_local, R, seed, row0, 0, dt, dev, out=S)
            e1.record()
            torch.cuda.synchronize()
            fill_ms = e0.elapsed_time(e1) / 20
            kernel = ("dense_pair_kernel (cta_group::2; dense_gemm_kernel where the tiles would not fill the CTA pairs): y = z S^T and "
                      "g = dY S, average over both launches, on S hashed once per call into a bf16 scratch by noise_bf16_seg_kernel "
                      "(noise_bf16x8_kernel when d_c is not a multiple of 1024)")
        else:
            avg_ms, fill_ms, kernel = fused_ms, None, fused["kernel"]
        achieved = flops_launch / (avg_ms * 1e-3) / 1e12
        # SM clock the dominant kernel actually ran at: cycles its MMA thread counted from first to last k-block, over the
        # launch's CUDA-event time (a lower bound: prologue and the last epilogue are outside the counted span); nvidia-smi
        # samples every 50 ms and mostly sees the idle clock
        sm_mhz_in_kernel = None
        if staged:
            try:
                from randumb_b200 import _lib
                prof = torch.zeros(148 * 16, dtype=torch.int64, device=dev)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                for _ in range(5):
                    K.gemm_dense(dy, S, True, False)
                _lib.lib().rdb_set_profile_buffer(prof.data_ptr(), prof.numel() * 8)
                e0.record()
                K.gemm_dense(dy, S, True, False)
                e1.record()
                torch.cuda.synchronize()
                _lib.lib().rdb_set_profile_buffer(None, 0)
                cyc = int(prof.view(148, 16)[:, 3].max().item())
                if cyc > 0:
                    sm_mhz_in_kernel = cyc / (e0.elapsed_time(e1) * 1e3)
            except Exception:
                sm_mhz_in_kernel = None
        roofline = {"bound": "tensor", "kernel": kernel, "achieved": achieved,
                    "peak": peaks["tensor"], "unit": "TFLOP/s", "frac": achieved / peaks["tensor"],
                    "peak_source": f"{peaks['src']} burst bf16", "avg_launch_ms": avg_ms,
                    "traffic": (DENSE_ON_NOISE_DRAM_BYTES if staged else NOISE_GEMM_DRAM_BYTES).get(args.workload),
                    "noise_fill_ms": fill_ms, "regenerate_in_kernel": fused if staged else None,
                    "sm_mhz_in_kernel": sm_mhz_in_kernel}
    else:
        # matrix-vector: bytes of C read twice and dC written once (+ the small vectors)
        bytes_step = 3 * R * Kin * 4 + 4 * (3 * Kin + 2 * N + 2 * R)
        achieved = bytes_step / (elapsed_ms / args.steps * 1e-3) / 1e9
        roofline = {"bound": "hbm", "kernel": "gemv_cx / gemv_sz / gemv_stdy / gemv_dxdc (whole step)", "achieved": achieved,
                    "peak": peaks["hbm"], "unit": "GB/s", "frac": achieved / peaks["hbm"], "peak_source": f"{peaks['src']} copy",
                    "traffic": None}

    # ---- end to end through the public module API, host buffers, copies inside the timed region ----
    e2e = run_e2e(args, cfg, rb, dev, world, dt, x_host, C, n_local, row0, barrier)
    if world > 1:
        e2e["host_placement"] = (f"rank 0 pinned to the cores of NUMA node {numa_node}, the node of its GPU (every rank likewise)"
                                 if numa_node is not None else "no NUMA placement exposed: ranks not pinned")

    if args.workload == "gemv":
        bytes_step = 3 * R * Kin * 4 + 4 * (3 * Kin + 2 * N + 2 * R)
        value = world * bytes_step * args.steps / (elapsed_ms * 1e-3) / 1e9
        unit = "GB/s"
    else:
        # data parallel: every rank does the whole layer on its own tokens; sharded: the ranks split ONE layer
        total = algorithmic_flops(T, Kin, N, R) * (world if args.workload == "gemm" else 1)
        value = total * args.steps / (elapsed_ms * 1e-3) / 1e12
        unit = "TFLOP/s"

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        torch.set_num_threads(os.cpu_count() or 1)
        T_s = pick_cpu_sample(cfg, budget_s=20.0)
        dt_cpu, _ = cpu_reference_step(cfg, T_s)
        if args.workload == "gemv":
            v = (3 * R * Kin * 4 + 4 * (3 * Kin + 2 * N + 2 * R)) / dt_cpu / 1e9
        else:
            v = algorithmic_flops(T_s, Kin, N, R) / dt_cpu / 1e12
        cpu_baseline = {"value": v, "unit": unit, "cores": torch.get_num_threads(), "cpu": cpu_model(), "kind": "port",
                        "sample": f"one step at {T_s} of {T} tokens (full K/N/d_c) in {dt_cpu:.2f} s: explicit S from the C oracle, "
                                  "W = S @ C, F.linear, autograd; float32"}

    if rank == 0:
        line = {
            "metric": metric_name(args.workload), "value": value, "unit": unit, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": elapsed_ms / args.steps, "higher_is_better": True,
            "scaling": "strong" if args.workload == "sharded" else "weak", "vs_baseline": None,
            "dtype": cfg["dtype"], "data": "synthetic",
            "config": dict(workload_config(args.workload, cfg, world, args.replicate_grads, args.gather_output),
                           **({"exchange": sb.exchange} if sb is not None else {})),
            "clocks": clocks, "e2e": e2e, "gpu_launches": (launches_per_step(args.workload, staged) + (5 if dc_sum is not None else 0)) * args.steps,   # + the peer-memory sum of dC: scatter, barrier, ordered sum, store, barrier
            "roofline": roofline, "cpu_baseline": cpu_baseline,
        }
        if step_ms:
            # this rank's per-step device times: median and the reference's 20 / 80 % quantiles (benchmark.py:50)
            q = lambda f: step_ms[min(len(step_ms) - 1, int(f * len(step_ms)))]
            line["ms_per_step_quantiles"] = {"p20": q(0.2), "median": q(0.5), "p80": q(0.8)}
        if eager_ms is not None:
            line["config"]["launch"] = "the step's four kernels replayed as one CUDA graph"
            line["eager_ms_per_step"] = eager_ms
    sharded = None
    if args.workload == "gemm" and not args.no_sharded_record:
        # the second scaling curve: the row-sharded layer on the same N GPUs, same steps and warm-up, same process
        del x, dy
        torch.cuda.empty_cache()
        sharded = sharded_record(args, dev, world, rank, rb, K)
    if rank == 0:
        if sharded is not None:
            line["sharded"] = sharded
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def launches_per_step(workload, staged):
    # forward: dense z + generated-operand y; backward: generated-operand g + dense dX + dense dC;
    # with S staged, forward and backward each launch the noise kernel once more
    if workload == "gemv":
        return 4
    return 7 if staged else 5


# DRAM bytes per launch of the generated-operand kernels: dram__bytes_read.sum + dram__bytes_write.sum of the
# ncu capture summarised under profiles/ (2048-token case, 70.7 MB), scaled by tokens to the 8192-token launch.
NOISE_GEMM_DRAM_BYTES = {"gemm": 2.83e8, "sharded": None}
# the same for the plain tensor-core products reading the staged S: 4096-token capture under profiles/, token-proportional
# terms doubled, average of the y-shaped (2.10e8) and g-shaped (3.11e8) launch
DENSE_ON_NOISE_DRAM_BYTES = {"gemm": 2.6e8, "sharded": None}


class _MeanSquare(torch.autograd.Function):
    """mean(y^2) with one reduction kernel forward (float32 accumulation over the bf16 values) and one elementwise kernel
    backward; the stock `y.float().square().mean()` spends more device time on float32 temporaries of y than the layer does."""

    @staticmethod
    def forward(ctx, y):
        ctx.save_for_backward(y)
        n = torch.linalg.vector_norm(y, dtype=torch.float32)
        return n * n / y.numel()

    @staticmethod
    def backward(ctx, grad):
        (y,) = ctx.saved_tensors
        return y * (grad * (2.0 / y.numel())).to(y.dtype)


def run_e2e(args, cfg, rb, dev, world, dt, x_host, C, n_local, row0, barrier):
    """Same step through RandumbLinear-style public API: x comes from pinned host memory every step
    (prefetched on a copy stream so the transfer overlaps the previous step's kernels), the loss value is
    read back to the host every step."""
    import torch.distributed as dist
    T, Kin, N, R, seed = cfg["T"], cfg["K"], cfg["N"], cfg["R"], cfg["seed"]
    coef = torch.nn.Parameter(C.clone())
    copy_stream = torch.cuda.Stream(device=dev)
    hosts = [x_host, x_host.clone().pin_memory()]
    bufs = [torch.empty_like(x_host, device=dev) for _ in range(2)]
    ready = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]

    def prefetch(i):
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(consumed[i % 2])
            bufs[i % 2].copy_(hosts[i % 2], non_blocking=True)
            ready[i % 2].record(copy_stream)

    def one(i, nsteps):
        torch.cuda.current_stream(dev).wait_event(ready[i % 2])
        if i + 1 < nsteps:
            prefetch(i + 1)
        xin = bufs[i % 2].requires_grad_(True)
        y = rb.rlinear(xin, coef, seed, n_local, row0)
        loss = _MeanSquare.apply(y)
        loss.backward()
        consumed[i % 2].record(torch.cuda.current_stream(dev))
        if world > 1:
            dist.all_reduce(coef.grad)
            if args.workload == "sharded":
                dist.all_reduce(xin.grad)              # every rank holds only its rows' contribution to dX
        val = float(loss.item())                       # device -> host read of the step's result
        coef.grad = None
        bufs[i % 2].requires_grad_(False)
        bufs[i % 2].grad = None
        return val

    n_e2e = max(3, min(args.steps, 10))
    for c in consumed:
        c.record(torch.cuda.current_stream(dev))
    prefetch(0)
    for i in range(3):
        one(i, 3)
    barrier()
    for c in consumed:
        c.record(torch.cuda.current_stream(dev))
    prefetch(0)
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for i in range(n_e2e):
        one(i, n_e2e)
    ev1.record()
    barrier()
    ms = ev0.elapsed_time(ev1)
    tmax = torch.tensor([ms], device=dev)
    if world > 1:
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
    ms = float(tmax.item())
    if args.workload == "gemv":
        work = world * (3 * R * Kin * 4 + 4 * (3 * Kin + 2 * N + 2 * R)) / 1e9
        unit = "GB/s"
    else:
        work = algorithmic_flops(T, Kin, N, R) * (world if args.workload == "gemm" else 1) / 1e12
        unit = "TFLOP/s"
    # the host -> device copy on its own, all ranks copying at the same time (what the end-to-end step is bound by when the
    # layer is faster than the copy): GB/s per rank, slowest rank
    h2d_bytes = x_host.numel() * x_host.element_size()
    barrier()
    c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    c0.record()
    for i in range(6):
        bufs[i % 2].copy_(hosts[i % 2], non_blocking=True)
    c1.record()
    barrier()
    tcopy = torch.tensor([c0.elapsed_time(c1) / 6], device=dev)
    if world > 1:
        dist.all_reduce(tcopy, op=dist.ReduceOp.MAX)
    copy_ms = float(tcopy.item())
    return {"value": work * n_e2e / (ms * 1e-3), "unit": unit, "h2d_bytes_per_step": h2d_bytes,
            "d2h_bytes_per_step": 4, "steps": n_e2e, "ms_per_step": ms / n_e2e,
            "h2d_gbs": h2d_bytes / (copy_ms * 1e-3) / 1e9, "h2d_copy_ms": copy_ms,
            "h2d_note": f"pinned-host -> device copy of one step's x alone, {world} rank(s) copying at once: the step cannot be shorter",
            "what": "pinned-host x -> device (copy stream, overlapped), rlinear forward, mean-square loss, autograd backward "
                    "(dX and dC), loss.item() back to the host"}


# --------------------------------------------------------------------------------------------------
# GPT-2-small-shaped workload: only the pseudorandom-weight layers of the 12 blocks (c_fc 768 -> 3072, c_proj 3072 -> 768,
# d_c = 128, seeds 13, 20, 27, ...), 8 x 1024 tokens per GPU, data parallel with one flat all-reduce of the 24 dC
# --------------------------------------------------------------------------------------------------
GPT2 = dict(T=8192, d=768, mlp=3072, R=128, blocks=12, seed0=13, seed_step=7, coef_std=(3 * 0.02 ** 2 / 128) ** 0.5)


def gpt2_whole_step(args, dev, world, rank, rb, randumb_ms):
    """One training step of a GPT-2-small-shaped model (12 pre-LN blocks, d 768, 12 heads, MLP 3072 with tanh-GELU, vocabulary
    50257, 8 x 1024 tokens per GPU) whose MLP projections are the pseudorandom-weight layers (d_c = 128, seeds 13 + 7 i); every
    other weight is a random bf16 tensor.  Forward, cross-entropy, backward, one flat all-reduce of the coefficient
    gradients, fused Adam on the coefficients.  Attention, layer norms and the dense projections are PyTorch's own kernels:
    this measures where the pseudorandom-weight layers sit in a step, not those kernels."""
    import torch.distributed as dist
    import torch.nn as nn
    import torch.nn.functional as F
    c = GPT2
    d, mlp, R, nb, heads, vocab, B, S = c["d"], c["mlp"], c["R"], c["blocks"], 12, 50257, 8, 1024
    dt = torch.bfloat16
    seeds = rb.stepgen(c["seed0"], c["seed_step"])

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.ln1, self.ln2 = nn.LayerNorm(d), nn.LayerNorm(d)
            self.qkv, self.proj = nn.Linear(d, 3 * d), nn.Linear(d, d)
            self.fc = rb.RandumbLinear(d, mlp, R, next(seeds), init_std=0.02)
            self.cproj = rb.RandumbLinear(mlp, d, R, next(seeds), init_std=0.02)

        def forward(self, x):
            b, s, _ = x.shape
            q, k, v = self.qkv(self.ln1(x)).view(b, s, 3, heads, d // heads).permute(2, 0, 3, 1, 4)
            a = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(b, s, d)
            x = x + self.proj(a)
            return x + self.cproj(F.gelu(self.fc(self.ln2(x)), approximate="tanh"))

    class Model(nn.Module):
        def __init__(self):
            super().__init__()
            self.wte, self.wpe = nn.Embedding(vocab, d), nn.Embedding(S, d)
            self.blocks = nn.ModuleList([Block() for _ in range(nb)])
            self.ln_f = nn.LayerNorm(d)
            self.lm_head = nn.Linear(d, vocab, bias=False)

        def forward(self, idx, targets):
            x = self.wte(idx) + self.wpe(torch.arange(idx.shape[1], device=idx.device))
            for blk in self.blocks:
                x = blk(x)
            logits = self.lm_head(self.ln_f(x))
            return F.cross_entropy(logits.float().view(-1, vocab), targets.view(-1))

    torch.manual_seed(1234)
    model = Model()
    for name, p in model.named_parameters():
        if not name.endswith("weight_coef") and p.dim() >= 2:
            nn.init.normal_(p, 0.0, 0.02)
    model = model.to(dev).to(dt)
    coefs = [p for n, p in model.named_parameters() if n.endswith("weight_coef")]
    g = torch.Generator().manual_seed(1004 + rank)
    idx_host = torch.randint(0, vocab, (B, S), generator=g).pin_memory()
    tgt_host = torch.randint(0, vocab, (B, S), generator=g).pin_memory()
    out = {}
    for variant in ("frozen", "all_trainable"):
        for n, p in model.named_parameters():
            p.requires_grad_(variant == "all_trainable" or n.endswith("weight_coef"))
            p.grad = None
        params = [p for p in model.parameters() if p.requires_grad]
        opt = torch.optim.Adam(params, lr=1e-4, fused=True)

        def step():
            idx = idx_host.to(dev, non_blocking=True)
            tgt = tgt_host.to(dev, non_blocking=True)
            loss = model(idx, tgt)
            loss.backward()
            if world > 1:
                rb.parallel.allreduce_coef_grads(params)          # one flat bucket: the coefficients, or every weight
            opt.step()
            opt.zero_grad(set_to_none=True)
            return loss

        for _ in range(3):
            loss = step()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        n = max(3, min(args.steps, 10))
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            loss = step()
        e1.record()
        first_loss = float(loss.item())
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / n], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        out[variant] = {"ms_per_step": ms, "tokens_per_s": world * B * S / (ms * 1e-3),
                        "trainable_parameters": sum(p.numel() for p in params), "loss": first_loss,
                        "pseudorandom_layers_share": randumb_ms / ms}
        del opt
    out["what"] = ("GPT-2-small-shaped step (12 blocks, d 768, 12 heads, MLP 3072, vocabulary 50257, 8 x 1024 tokens per GPU): forward, "
                   "cross-entropy, backward, flat gradient all-reduce, fused Adam; 'frozen' trains the 24 coefficient matrices only (the "
                   "all-reduce carries only dC), 'all_trainable' every weight.  pseudorandom_layers_share = the 24 layers' own time "
                   "(this line's ms_per_step) over the whole step; the rest is PyTorch's attention, layer norms, dense projections, "
                   "embedding and loss kernels")
    out["expected_initial_loss"] = "about ln(50257) = 10.82 for random weights (modded-nanogpt/train_gpt2.py:241 of the reference)"
    return out


def run_gpt2mlp(args):
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py measures the CUDA kernels; no GPU is visible (there is no CPU fallback)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        if os.environ.get("NCCL_DEBUG", "VERSION").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"
        dist.init_process_group("nccl", device_id=dev)
    from randumb_b200 import kernels as K
    import randumb_b200 as rb
    c = GPT2
    T, d, mlp, R, nb = c["T"], c["d"], c["mlp"], c["R"], c["blocks"]
    dt = torch.bfloat16
    g = torch.Generator().manual_seed(1004 + rank)
    x1_host = torch.randn(T, d, generator=g).to(dt).pin_memory()
    x1, x2 = x1_host.to(dev), torch.randn(T, mlp, generator=g).to(dt).to(dev)
    dy1, dy2 = torch.randn(T, mlp, generator=g).to(dt).to(dev), torch.randn(T, d, generator=g).to(dt).to(dev)
    gc = torch.Generator().manual_seed(7)
    layers = []                                   # (x, dy, coef, seed, out_features)
    for b in range(nb):
        s_fc, s_proj = c["seed0"] + c["seed_step"] * (2 * b), c["seed0"] + c["seed_step"] * (2 * b + 1)
        layers.append((x1, dy1, (torch.randn(R, d, generator=gc) * c["coef_std"]).to(dt).to(dev), s_fc, mlp))
        layers.append((x2, dy2, (torch.randn(R, mlp, generator=gc) * c["coef_std"]).to(dt).to(dev), s_proj, d))
    flops_step = sum(algorithmic_flops(T, L[0].shape[1], L[4], R) for L in layers)

    def compute():
        dcs = []
        for x, dy, C, seed, n_out in layers:
            K.linear_fwd(x, C, seed, n_out)
        for x, dy, C, seed, n_out in reversed(layers):
            dx, dc = K.linear_bwd(dy, x, C, seed)
            dcs.append(dc.reshape(-1))
        return torch.cat(dcs)                     # 5.9 M coefficients, 11.8 MB bf16

    # 216 short launches per step: replayed as one CUDA graph so that the host's launch rate is not what is measured
    # (the all-reduce stays outside the graph, on the graph's output buffer)
    graph, flat_static = None, None
    if not args.no_graph:
        for _ in range(2):
            compute()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            flat_static = compute()

    def step():
        if graph is not None:
            graph.replay()
            flat = flat_static
        else:
            flat = compute()
        if world > 1:
            dist.all_reduce(flat)
        return flat

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.15)
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_wall0 = time.time()
    ev0.record()
    for _ in range(args.steps):
        step()
    ev1.record()
    barrier()
    t_wall1 = time.time()
    clocks = sampler.stop(t_wall0, t_wall1) if rank == 0 else None
    K.check_status()
    tmax = torch.tensor([ev0.elapsed_time(ev1)], device=dev)
    if world > 1:
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
    elapsed_ms = float(tmax.item())
    value = world * flops_step * args.steps / (elapsed_ms * 1e-3) / 1e12

    # end to end: the MLP halves of the 12 blocks as modules (residual stream, tanh-GELU), x from pinned host memory,
    # autograd backward, the loss value read back
    seeds = rb.stepgen(c["seed0"], c["seed_step"])
    blocks = [(rb.RandumbLinear(d, mlp, R, next(seeds), device=dev, dtype=dt), rb.RandumbLinear(mlp, d, R, next(seeds), device=dev, dtype=dt))
              for _ in range(nb)]
    params = [m.weight_coef for pair in blocks for m in pair]
    xin = torch.empty_like(x1)

    def e2e_step():
        xin.copy_(x1_host, non_blocking=True)
        h = xin
        for fc, proj in blocks:
            h = h + proj(torch.nn.functional.gelu(fc(h), approximate="tanh"))
        loss = _MeanSquare.apply(h)
        loss.backward()
        if world > 1:
            rb.parallel.allreduce_coef_grads(params)
        val = float(loss.item())
        for p_ in params:
            p_.grad = None
        return val

    for _ in range(3):
        e2e_step()
    barrier()
    n_e2e = max(3, min(args.steps, 10))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n_e2e):
        e2e_step()
    e1.record()
    barrier()
    t2 = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if world > 1:
        dist.all_reduce(t2, op=dist.ReduceOp.MAX)
    e2e_ms = float(t2.item()) / n_e2e
    e2e = {"value": world * flops_step / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": x1_host.numel() * 2,
           "d2h_bytes_per_step": 4, "steps": n_e2e, "ms_per_step": e2e_ms,
           "what": "pinned-host x -> device, 12 x (RandumbLinear, tanh-GELU, RandumbLinear, residual), mean-square loss, autograd "
                   "backward, flat dC all-reduce, loss.item(); TFLOP/s counts the pseudorandom-weight layers only"}

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        torch.set_num_threads(os.cpu_count() or 1)
        dt_cpu, fl_cpu = 0.0, 0.0
        for (Kin, n_out, seed) in ((d, mlp, c["seed0"]), (mlp, d, c["seed0"] + c["seed_step"])):
            cc = dict(T=T, K=Kin, N=n_out, R=R, seed=seed, dtype="bf16", coef_std=c["coef_std"])
            cpu_reference_step(cc, T)
            t_, _ = cpu_reference_step(cc, T)
            dt_cpu += t_
            fl_cpu += algorithmic_flops(T, Kin, n_out, R)
        cpu_baseline = {"value": fl_cpu / dt_cpu / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "cpu": cpu_model(), "kind": "port",
                        "sample": f"one block's two layers (of 12 blocks) at all {T} tokens in {dt_cpu:.2f} s: explicit S from the C "
                                  "oracle, W = S @ C, F.linear, autograd; float32"}
    whole = None
    if not args.no_whole_step:
        del blocks, params
        torch.cuda.empty_cache()
        whole = gpt2_whole_step(args, dev, world, rank, rb, elapsed_ms / args.steps)
    if rank == 0:
        peaks = measured_peaks()
        per_gpu = value / world
        line = {
            "metric": metric_name("gpt2mlp"), "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": elapsed_ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"gpt2mlp: the 24 pseudorandom-weight layers of GPT-2 small's 12 MLPs (768 -> 3072 -> 768, d_c=128, "
                                   f"seeds {c['seed0']}+{c['seed_step']}i), {T} tokens per GPU, fwd + dX + dC of every layer",
                       "parallelism": f"dp{world} (one flat all-reduce of the 24 dC, 11.8 MB)" if world > 1 else "single GPU",
                       "launch": "eager launches" if graph is None else "the step's 216 kernels replayed as one CUDA graph",
                       "l2": "one step streams about 1.5 GB of activations, outputs and gradients (24 layers), far more than the 126 MB L2 "
                             "(no explicit flush)"},
            "clocks": clocks, "e2e": e2e, "gpu_launches": 12 * 18 * args.steps,   # per block: c_fc fwd 3, c_proj fwd 4 (z split-K), c_proj bwd 5, c_fc bwd 6
            "roofline": {"bound": "tensor", "kernel": "whole step (24 layers, 216 launches; contractions of 128 and 768-8192)",
                         "achieved": per_gpu, "peak": peaks["tensor"], "unit": "TFLOP/s", "frac": per_gpu / peaks["tensor"],
                         "peak_source": f"{peaks['src']} burst bf16", "traffic": None},
            "cpu_baseline": cpu_baseline,
        }
        if whole is not None:
            line["whole_step"] = whole
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# --------------------------------------------------------------------------------------------------
# small cases for profilers (`--profile-case`): a few launches of one kind of kernel, then exit
# --------------------------------------------------------------------------------------------------
ROLE_NAMES = ["mma_wait_full_or_A", "mma_wait_B", "mma_wait_tmem", "mma_total", "tma_wait_free", "gen_wait_free", "gen_busy",
              "epilogue_busy"]


def profile_case(args):
    """Self-terminating cases sized for `ncu` (device footprint a few hundred MB, launches of 0.01-0.3 ms):

        --profile-case noise     2 launches each of the y- and g-shaped product with S regenerated in the kernel (-k regex:noise_)
        --profile-case staged    2 x (noise fill + plain product) for y and g on the staged S (-k "regex:dense_|noise_bf16")
        --profile-case products  2 launches each of the five plain products of one step (z, y, g, dX, dC)
        --profile-case gemv      3 forward + backward steps of the batch-1 float32 layer, L2 flushed in between (-k regex:gemv)
        --profile-case roles     per-role cycle counters of the generated-operand kernel variants and of the pair kernel
        --profile-case overlap   the noise fill beside the z product against one after the other
        --profile-case formr     materialise forward / backward and embedding rows of the 1-D-coefficient form, in hashes per second
        --profile-case hash      throughput of alternative formulations of the hash, each checked bit for bit (randumb_b200/lab)
      with --tokens / --out / --dc for the shape (defaults 2048 / 4096 / 8192 tokens, 16384 rows, d_c 1024).
    """
    from randumb_b200 import kernels as K, _lib
    assert torch.cuda.is_available(), "profile cases run on a GPU"
    case, out, dc, seed = args.profile_case, args.out, args.dc, 42
    if case == "hash":
        # alternative formulations of the hash (randumb_b200/lab/hash_variants.cu): compile with nvcc, run, print its table
        from randumb_b200 import build as _build
        src = os.path.join(ROOT, "randumb_b200", "lab", "hash_variants.cu")
        exe = os.path.join(ROOT, "randumb_b200", "lib", "hash_variants")
        os.makedirs(os.path.dirname(exe), exist_ok=True)
        subprocess.run([_build._nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-o", exe, src], check=True)
        subprocess.run([exe], check=True)
        print("ok")
        return
    if case == "formr":
        # the reference's own parameterisation (1-D coefficient vector): materialise forward / backward of a GPT-2-small MLP
        # weight and of an embedding lookup, against the rate of the bare hash loop (`--profile-case hash`)
        dev = torch.device("cuda", 0)

        def med(f, reps=10):
            for _ in range(2):
                f()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                f()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / reps

        for (P, Q, M) in ((3072, 768, 256), (3072, 768, 128), (50304, 768, 256)):
            coef = torch.randn(M, device=dev)
            dout = torch.randn(P * Q, device=dev)
            t_f = med(lambda: K.materialize_fwd(coef, [P, Q], [Q, 1], 13), reps=5 if P > 10000 else 10)
            t_b = med(lambda: K.materialize_bwd(dout, M, 13), reps=5 if P > 10000 else 10)
            h = P * Q * M
            print(f"weight [{P} x {Q}], int_dim {M}: {h / 1e9:.2f} G hashes per pass; materialize_fwd {t_f:.3f} ms = {h / (t_f * 1e-3) / 1e9:.0f} G hashes/s, "
                  f"materialize_bwd {t_b:.3f} ms = {h / (t_b * 1e-3) / 1e9:.0f} G hashes/s", flush=True)
        idx = torch.randint(0, 50304, (8 * 1024,), device=dev)
        coef = torch.randn(256, device=dev)
        t_e = med(lambda: K.embed_fwd(idx, coef, 768, 9))
        h = idx.numel() * 768 * 256
        print(f"embedding rows: 8192 tokens x 768, int_dim 256: {h / 1e9:.2f} G hashes; embed_fwd {t_e:.3f} ms = {h / (t_e * 1e-3) / 1e9:.0f} G hashes/s")
        print("ok")
        return
    if case == "overlap":
        # the noise fill beside the z product (a stream of its own) against the two in a row, at three shapes
        side = torch.cuda.Stream()

        def med(f, reps=20):
            for _ in range(3):
                f()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                f()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / reps * 1e3

        for (T, Kin, R, nloc, tag) in ((512, 16384, 2048, 8192, "token slice of the row-sharded layer at 8 ranks"),
                                       (2048, 16384, 2048, 32768, "the same at 2 ranks"), (8192, 4096, 1024, 16384, "headline layer")):
            x = torch.randn(T, Kin, device="cuda").bfloat16()
            C = (torch.randn(R, Kin, device="cuda") * 0.01).bfloat16()
            S = torch.empty(nloc, R, device="cuda", dtype=torch.bfloat16)
            z = torch.empty(T, R, device="cuda", dtype=torch.bfloat16)
            prod = lambda: K.gemm_dense(x, C, out=z)
            fill = lambda: K.noise(nloc, R, 7, 0, 0, out=S)

            def serial():
                fill(); prod()

            def beside():
                cur = torch.cuda.current_stream()
                side.wait_stream(cur)
                with torch.cuda.stream(side):
                    fill()
                prod()
                cur.wait_stream(side)
            print(f"{tag}: z = x C^T [{T} x {R}, contraction {Kin}] {med(prod):.1f} us, fill of S [{nloc} x {R}] {med(fill):.1f} us, "
                  f"one after the other {med(serial):.1f} us, fill on a second stream beside the product {med(beside):.1f} us", flush=True)
        print("ok")
        return
    if case == "grads":
        # dX = g C and dC = g^T x of rdb_linear_bwd one after the other and side by side on disjoint CTA pairs, at two shapes
        from randumb_b200 import _lib

        def med(f, reps=30):
            for _ in range(5):
                f()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                f()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / reps * 1e3

        for (T, Kin, N, R, tag) in ((8192, 4096, 16384, 1024, "headline layer"), (4096, 16384, 8192, 2048, "one of eight row shards of the 65536 x 16384 layer")):
            gen = torch.Generator().manual_seed(5)
            x = torch.randn(T, Kin, generator=gen).bfloat16().cuda()
            C = (torch.randn(R, Kin, generator=gen) * 0.02).bfloat16().cuda()
            dy = torch.randn(T, N, generator=gen).bfloat16().cuda()
            gg = torch.randn(T, R, generator=gen).bfloat16().cuda()
            bwd = lambda o: med(lambda: K.linear_bwd(dy, x, C, 1, 0, options=o))
            pairs = _lib.CallOptions(dense_pair=2)
            print(f"{tag} (T {T}, K {Kin}, N {N}, d_c {R}): rdb_linear_bwd one after the other {bwd(_lib.CallOptions(grads_beside=0)):.1f} us, "
                  f"automatic {bwd(None):.1f} us, side by side forced {bwd(_lib.CallOptions(grads_beside=2)):.1f} us; alone: "
                  f"dX {med(lambda: K.gemm_dense(gg, C, True, False)):.1f} us (CTA pairs {med(lambda: K.gemm_dense(gg, C, True, False, options=pairs)):.1f}), "
                  f"dC {med(lambda: K.gemm_dense(gg, x, False, False)):.1f} us (CTA pairs {med(lambda: K.gemm_dense(gg, x, False, False, options=pairs)):.1f})",
                  flush=True)
        K.check_status()
        print("ok")
        return
    tokens = args.tokens or {"noise": 2048, "staged": 4096, "products": 4096, "roles": 8192, "gemv": 1}[case]
    dev = torch.device("cuda", 0)
    if case == "gemv":
        cfg = WORKLOADS["gemv"]
        g = torch.Generator().manual_seed(1002)
        x = torch.randn(1, cfg["K"], generator=g).to(dev)
        C = (torch.randn(cfg["R"], cfg["K"], generator=g) * cfg["coef_std"]).to(dev)
        dy = torch.randn(1, cfg["N"], generator=g).to(dev)
        flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
        for _ in range(3):
            flush.zero_()
            K.linear_fwd(x, C, cfg["seed"], cfg["N"])
            K.linear_bwd(dy, x, C, cfg["seed"])
        torch.cuda.synchronize()
        print("ok")
        return
    z = torch.randn(tokens, dc, device=dev).bfloat16()
    dy = torch.randn(tokens, out, device=dev).bfloat16()
    if case == "noise":
        for _ in range(2):
            K.gemm_noise(z, out, seed, False, impl=K.IMPL_UMMA)       # y = z S^T
            K.gemm_noise(dy, dc, seed, True, impl=K.IMPL_UMMA)        # g = dY S
    elif case == "staged":
        assert K.linear_stages_noise(tokens, 8, out, dc, torch.bfloat16, K.PATH_FACTORED)
        for _ in range(2):
            K.noise_product(z, out, seed, False)       # noise fill + y = z S^T
            K.noise_product(dy, dc, seed, True)        # noise fill + g = dY S
    elif case == "products":
        kin = 4096
        x = torch.randn(tokens, kin, device=dev).bfloat16()
        C = (torch.randn(dc, kin, device=dev) * 0.01).bfloat16()
        S = K.noise(out, dc, seed, 0, 0, torch.bfloat16, dev)
        for _ in range(2):
            K.gemm_dense(x, C)                         # z = x C^T
            K.gemm_dense(z, S)                         # y = z S^T
            K.gemm_dense(dy, S, True, False)           # g = dY S
            K.gemm_dense(z, C, True, False)            # dX = g C
            K.gemm_dense(z, x, False, False)           # dC = g^T x
    else:
        L = _lib.lib()
        prof = torch.zeros(148 * 16, dtype=torch.int64, device=dev)
        S = K.noise(out, dc, seed, 0, 0, torch.bfloat16, dev)

        def counters(label, fn):
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(5):
                fn()
            e1.record()
            torch.cuda.synchronize()
            prof.zero_()
            L.rdb_set_profile_buffer(prof.data_ptr(), prof.numel() * 8)
            fn()
            torch.cuda.synchronize()
            L.rdb_set_profile_buffer(None, 0)
            p = prof.view(148, 16).double()[:, :8]
            issuing = p[p[:, 3] > 0]
            total = float(issuing[:, 3].mean())
            vals = issuing.mean(0)
            gens = p[p[:, 6] > 0]
            if gens.numel():
                vals[4:7] = gens.mean(0)[4:7]
            print(f"{label}: {e0.elapsed_time(e1) / 5:.4f} ms  mma_total {total / 1e3:.0f} kcycles  " +
                  "  ".join(f"{n}={100 * float(v) / total:.0f}%" for n, v in zip(ROLE_NAMES, vals.tolist())), flush=True)

        for tile in (1, 3, 7, 8):
            prev = K.set_option(_lib.OPT_NOISE_TILE, tile)
            try:
                counters(f"generated-operand variant {tile} y", lambda: K.gemm_noise(z, out, seed, False, impl=K.IMPL_UMMA))
                counters(f"generated-operand variant {tile} g", lambda: K.gemm_noise(dy, dc, seed, True, impl=K.IMPL_UMMA))
            finally:
                K.set_option(_lib.OPT_NOISE_TILE, prev)
        pair = _lib.CallOptions(dense_pair=2)
        counters("pair kernel y = z S^T", lambda: K.gemm_dense(z, S, options=pair))
        # the pair kernel's first epilogue warp of each CTA also counts, summed over its tiles: accumulator 0 seen complete ->
        # handed back [5], -> accumulator 1 handed back [6], store phase [7]
        ep = prof.view(148, 16).double()
        tiles_per_pair = -(-((tokens + 511) // 512) * ((out + 255) // 256) // 74)
        print(f"  per tile ({tiles_per_pair} tiles per pair), cycles: MMA thread waiting for TMEM {float(ep[::2, 2].mean()) / tiles_per_pair:.0f}; "
              f"epilogue warp, even / odd CTA: accumulator 0 complete -> handed back {float(ep[::2, 5].mean()) / tiles_per_pair:.0f} / "
              f"{float(ep[1::2, 5].mean()) / tiles_per_pair:.0f}, -> accumulator 1 handed back {float(ep[::2, 6].mean()) / tiles_per_pair:.0f} / "
              f"{float(ep[1::2, 6].mean()) / tiles_per_pair:.0f}, store phase {float(ep[::2, 7].mean()) / tiles_per_pair:.0f} / "
              f"{float(ep[1::2, 7].mean()) / tiles_per_pair:.0f}", flush=True)
        counters("pair kernel g = dY S", lambda: K.gemm_dense(dy, S, True, False, options=pair))
    torch.cuda.synchronize()
    K.check_status()
    print("ok")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="gemm", choices=list(WORKLOADS) + ["gpt2mlp"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--gather-output", action="store_true",
                    help="sharded workload: all-gather y (537 MB at the full size) so that every rank holds all of it")
    ap.add_argument("--replicate-grads", action="store_true",
                    help="sharded workload: all-gather dX and all-reduce dC so that every rank holds both in full")
    ap.add_argument("--no-graph", action="store_true", help="gemv workload: launch the four kernels eagerly in the timed region")
    ap.add_argument("--no-whole-step", action="store_true",
                    help="gpt2mlp workload: skip the `whole_step` sub-record (the full GPT-2-small-shaped training step around the layers)")
    ap.add_argument("--no-sharded-record", action="store_true",
                    help="default workload: skip the `sharded` sub-record (the row-sharded 65536 x 16384 layer measured after the headline)")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                    help="row-sharded layer: exchanges by the library's kernels over peer memory (falls back to NCCL when the ranks "
                         "cannot map each other's memory) or by NCCL collectives")
    ap.add_argument("--profile-case", default=None, choices=["noise", "staged", "roles", "products", "gemv", "hash", "overlap", "formr", "grads"],
                    help="run a small self-terminating case for a profiler instead of the benchmark")
    ap.add_argument("--tokens", type=int, default=None, help="profile case: token count")
    ap.add_argument("--out", type=int, default=16384, help="profile case: output rows")
    ap.add_argument("--dc", type=int, default=1024, help="profile case: coefficient dimension")
    args = ap.parse_args()
    if args.profile_case:
        profile_case(args)
        return
    if args.workload == "gpt2mlp" and args.impl == "ours":
        run_gpt2mlp(args)
        return
    cfg = WORKLOADS["gemm" if args.workload == "gpt2mlp" else args.workload]
    if args.impl == "reference":
        run_reference(args, cfg)
    else:
        run_ours(args, cfg)


if __name__ == "__main__":
    main()
