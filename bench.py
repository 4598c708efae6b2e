#!/usr/bin/env python
"""Benchmark of the preprocessing hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--no-extras]

Headline workload (one "step" = one pass of the resampler over one batch): bf16 trajectory
resampling, B=4096 rows per GPU, S=500, D=256, T=250 sorted-uniform target times per row, seeded
synthetic inputs resident in HBM.  ``value`` is GB/s over the bytes a resampler must move (the
smaller of "every tensor once" and "touched source rows + times + output").  Under torchrun each
rank owns its own B=4096 shard (weak scaling, no data-path collective); the time is the max over
ranks of the CUDA-event time of the K timed steps.

The line also carries: the HBM roofline of the resample kernel measured live, the end-to-end rate
from pinned host buffers through the public API, the CPU oracle timed on the host cores
(``cpu_baseline``), SM clocks sampled during the run, and — unless ``--no-extras`` — fusion and
voxelisation figures for the other headline configurations.

``--impl reference`` times the CPU restatement of the reference's torch path (the oracle port,
all host threads) on a bounded sample of the same workload and prints the same line shape.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

HEADLINE = dict(B=4096, S=500, D=256, T=250)
EXTRAS_LIMIT_S = 420          # multi-GPU runs: the side measurements get this long before the line is printed without them
METRIC = "resample_throughput"
UNIT = "GB/s"
WORKLOAD = "resample bf16 B=4096 S=500 D=256 T=250 sorted-uniform targets, per GPU"
RESAMPLE_DRAM_BYTES_PER_ROW = (169117952 + 88358656) / 1024   # ncu capture, B=1024
BYTES_CONVENTION = "min(all tensors once, touched rows + times + output)"


# ----------------------------------------------------------------------------- helpers

def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(prefix="clocks_", suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, smax, reasons, power = [], [], set(), []
        try:
            for line in open(self.path):
                p = [x.strip() for x in line.split(",")]
                if len(p) < 9 or not p[0].isdigit() or int(p[0]) != self.gpu_index:
                    continue
                try:
                    sm.append(float(p[1])); smax.append(float(p[2])); power.append(float(p[3]))
                except ValueError:
                    continue
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), p[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        # samples under load: the upper half by power draw
        if sm:
            order = sorted(range(len(sm)), key=lambda i: power[i])
            loaded = [sm[i] for i in order[len(order) // 2:]]
        else:
            loaded = []
        return {"sm_mhz": statistics.median(loaded) if loaded else None,
                "sm_max_mhz": max(smax) if smax else None, "reasons": sorted(reasons), "samples": len(sm)}


def host_threads() -> int:
    """Host cores this process may use (torchrun pins OMP_NUM_THREADS=1, which is not what is wanted here)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return os.cpu_count() or 1


def physical_gpu_index(local_rank: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except Exception:
            return local_rank
    return local_rank


class LineGuard:
    """Prints the benchmark's one JSON line exactly once: normally from ``finish()``; from a timer thread if
    ``limit_s`` seconds pass first (the main thread may then be stuck inside a collective), after which the
    process ends with status 0.  ``printer`` is False on the ranks that print nothing; their timer only ends them."""

    def __init__(self, printer: bool, build_line, extras: dict, limit_s):
        self.printer, self.build_line, self.extras, self.limit_s = printer, build_line, extras, limit_s
        self._once = threading.Lock()
        self._timer = None

    def _emit(self):
        if self._once.acquire(blocking=False) and self.printer:
            print(json.dumps(self.build_line()), flush=True)

    def _give_up(self):
        self.extras["watchdog"] = f"side measurements did not finish within {self.limit_s} s; line printed without the rest"
        self._emit()
        sys.stdout.flush()
        os._exit(0)

    def start(self):
        if self.limit_s is not None:
            self._timer = threading.Timer(self.limit_s, self._give_up)
            self._timer.daemon = True
            self._timer.start()

    def finish(self):
        if self._timer is not None:
            self._timer.cancel()
        self._emit()


def dist_setup(n_gpus: int):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        # The watchdog of the side measurements may end the processes abruptly, and a process that dies while NCCL has
        # memory bound to an NVLink multicast object can fault the other GPUs: leave the in-switch reduction off.  The
        # headline path has no data-path collective; the grid-reduce side measurements run without NVLS.
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    else:
        torch.cuda.set_device(local)
    return rank, world, local


def max_over_ranks(ms: float, world: int, dev) -> float:
    if world == 1:
        return ms
    import torch.distributed as dist
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def barrier(world: int):
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()


def timed_region(step, steps: int, warmup: int, world: int, dev):
    """W untimed steps, then K steps between events; returns (max-over-ranks total ms, per-step ms list)."""
    for _ in range(warmup):
        step()
    barrier(world)
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    evs[0].record()
    for k in range(steps):
        step()
        evs[k + 1].record()
    torch.cuda.synchronize()
    barrier(world)
    total = evs[0].elapsed_time(evs[-1])
    per = [evs[k].elapsed_time(evs[k + 1]) for k in range(steps)]
    return max_over_ranks(total, world, dev), per


class L2Flush:
    """Writes a buffer larger than L2 so the next timed call starts from DRAM."""
    def __init__(self, dev, nbytes=256 << 20):
        self.buf = torch.empty(nbytes, dtype=torch.uint8, device=dev)

    def __call__(self):
        self.buf.zero_()


def time_cold(fn, iters: int, warmup: int, flush: L2Flush):
    """Median and mean of per-call CUDA-event times with an L2 flush before every call (ms)."""
    for _ in range(warmup):
        flush(); fn()
    ts = []
    for _ in range(iters):
        flush()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(); fn(); b.record()
        b.synchronize()
        ts.append(a.elapsed_time(b))
    return statistics.median(ts), sum(ts) / len(ts)


# ----------------------------------------------------------------------------- reference arm

def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle
    from robogoat_b200 import workloads
    threads = host_threads()
    B_s = 256                                  # bounded sample: 1/16 of the headline batch per step
    src, st, tt = workloads.resample_inputs(B=B_s, dtype=torch.bfloat16, irregular_targets=True, seed=0,
                                            S=HEADLINE["S"], D=HEADLINE["D"], T=HEADLINE["T"])
    left, right, _ = oracle.brackets(st, tt)
    nbytes = min(workloads.resample_bytes(B_s, HEADLINE["S"], HEADLINE["T"], HEADLINE["D"], 2),
                 workloads.resample_touched_bytes(left, right, HEADLINE["S"], HEADLINE["D"], 2))
    for _ in range(max(args.warmup, 1)):
        oracle.resample_trajectories(src, st, tt, threads=threads)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle.resample_trajectories(src, st, tt, threads=threads)
    dt = time.perf_counter() - t0
    gbs = nbytes * args.steps / dt / 1e9
    sample = f"B={B_s} rows of the B=4096 headline batch per step (same S, D, T, generator), oracle port, {threads} threads"
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": "B=256 rows per step (the CPU rate does not depend on B)",
                   "bytes_per_step": nbytes, "bytes_convention": BYTES_CONVENTION},
        "cpu_baseline": {"value": gbs, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": gbs, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    ref_gpu = reference_cuda_leg()
    if ref_gpu is not None:
        line["reference_cuda_kernels_on_this_gpu"] = ref_gpu
    print(json.dumps(line), flush=True)


def reference_cuda_leg():
    """Context for the reference arm: the reference's own CUDA kernels (compiled unmodified for sm_100a into
    oracle/_ref with its flags) timed with CUDA events on the same workloads.  None where the library or a GPU
    is missing.  Their outputs differ from the parity target outside the source time range (they extrapolate)."""
    try:
        import oracle
        from robogoat_b200 import workloads
        if oracle.ref_cuda_lib() is None or not torch.cuda.is_available():
            return None
        dev = torch.device("cuda", 0)
        torch.cuda.set_device(0)

        def timed(fn, n):
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(n):
                fn()
            b.record(); torch.cuda.synchronize()
            return a.elapsed_time(b) / n

        out = {}
        B, S, D, T = HEADLINE["B"], HEADLINE["S"], HEADLINE["D"], HEADLINE["T"]
        src, st, tt = workloads.resample_inputs(B=B, S=S, D=D, T=T, dtype=torch.bfloat16, irregular_targets=True, seed=0, device=dev)
        o = torch.empty((B, T, D), dtype=torch.bfloat16, device=dev)
        ms = timed(lambda: oracle.ref_cuda_resample(src, st, tt, out=o), 10)
        out["resample_bf16_B4096"] = {"ms": ms, "GB/s_all_tensors_once": workloads.resample_bytes(B, S, T, D, 2) / (ms * 1e-3) / 1e9}
        del src, o
        a = workloads.fusion_inputs(B=16384, dtype=torch.bfloat16, seed=0, device=dev)
        o = torch.empty((16384, 50, 588), dtype=torch.bfloat16, device=dev)
        ms = timed(lambda: oracle.ref_cuda_fuse(*a, out=o), 10)
        out["fusion_bf16_B16384"] = {"ms": ms, "GB/s": workloads.fusion_bytes(16384, 50, 2) / (ms * 1e-3) / 1e9}
        del a, o
        pts = workloads.voxel_uniform_inputs(500_000, seed=0, device=dev)
        kw = workloads.VOXEL_OCCUPANCY_GEOMETRY
        ms = timed(lambda: oracle.ref_cuda_voxelize(pts, None, kw["grid_min"], kw["voxel_size"], kw["grid_size"], "occupancy"), 50)
        out["voxel_occupancy_500k_128"] = {"us": ms * 1e3, "Gpts/s": 500_000 / (ms * 1e-3) / 1e9, "note": "warm L2, zero-fill by torch included"}
        N = 1 << 26
        pts, feats = workloads.voxel_mixture_inputs(N, seed=0, device=dev)
        kw = workloads.VOXEL_MIXTURE_GEOMETRY
        for mode in ("count", "mean"):
            ms = timed(lambda: oracle.ref_cuda_voxelize(pts, feats if mode == "mean" else None, kw["grid_min"], kw["voxel_size"],
                                                        kw["grid_size"], mode), 5)
            out[f"voxel_{mode}_64M_512"] = {"ms": ms, "Gpts/s": N / (ms * 1e-3) / 1e9}
        return out
    except Exception as e:  # a comparator must never break the arm
        return {"error": repr(e)}


# ----------------------------------------------------------------------------- our arm

def run_ours(args):
    from robogoat_b200 import _lib, ops, workloads
    import robocache

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path to measure)")
    L = _lib.load()
    rank, world, local = dist_setup(args.gpus)
    dev = torch.device("cuda", local)
    B, S, D, T = HEADLINE["B"], HEADLINE["S"], HEADLINE["D"], HEADLINE["T"]

    src, st, tt = workloads.resample_inputs(B=B, S=S, D=D, T=T, dtype=torch.bfloat16, irregular_targets=True,
                                            seed=rank, device=dev)
    out = torch.empty((B, T, D), dtype=torch.bfloat16, device=dev)
    left, right, _ = ops.resample_brackets_cuda(st, tt)
    algo_bytes = workloads.resample_bytes(B, S, T, D, 2)
    touched_bytes = workloads.resample_touched_bytes(left, right, S, D, 2)
    step_bytes = min(algo_bytes, touched_bytes)
    del left, right
    stream = torch.cuda.current_stream(dev).cuda_stream

    def step():
        rc = L.rc_resample(src.data_ptr(), st.data_ptr(), tt.data_ptr(), out.data_ptr(), B, S, T, D, _lib.RC_DTYPE_BF16,
                           local, stream)
        if rc != 0:
            raise RuntimeError(f"rc_resample failed: {rc}")

    sampler = ClockSampler(physical_gpu_index(local))
    if rank == 0:
        sampler.start()
    total_ms, per = timed_region(step, args.steps, args.warmup, world, dev)
    # keep the kernel running long enough for the clock sampler to see it under load
    if rank == 0:
        t_end = time.time() + 1.0
        while time.time() < t_end:
            for _ in range(50):
                step()
            torch.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 else None
    barrier(world)

    ms_per_step = total_ms / args.steps
    value = step_bytes * world / (ms_per_step * 1e-3) / 1e9
    kernel_ms = statistics.mean(per)
    peak, peak_kind = measured_peak_gbs()
    achieved = step_bytes / (kernel_ms * 1e-3) / 1e9
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": int(RESAMPLE_DRAM_BYTES_PER_ROW * B), "traffic_source": "ncu dram__bytes_read+write of a B=1024 capture (profiles/resample_gather_bf16_B1024.md), scaled by rows", "peak_source": f"of {peak_kind}", "kernel": "interp_gather_kernel<bf16, 16 B, staged, uniform>",
                "kernel_ms": kernel_ms, "bytes_algorithmic_all_tensors_once": algo_bytes,
                "bytes_touched_rows": touched_bytes, "achieved_all_tensors_once": algo_bytes / (kernel_ms * 1e-3) / 1e9}

    # ---- end to end through the public API: pinned host inputs -> device -> op -> pinned host output
    e2e_steps = max(3, min(args.steps, 10))
    h_src, h_st, h_tt = src.cpu().pin_memory(), st.cpu().pin_memory(), tt.cpu().pin_memory()
    h_out = torch.empty((B, T, D), dtype=torch.bfloat16).pin_memory()

    from robogoat_b200.host_pipeline import resample_trajectories_host

    def e2e_step():
        # host-buffer entry point of the package: chunked upload / kernel / download on three streams
        resample_trajectories_host(h_src, h_st, h_tt, out=h_out, device=dev, chunk_rows=256)

    e2e_ms, _ = timed_region(e2e_step, e2e_steps, 2, world, dev)
    e2e_val = step_bytes * world / (e2e_ms / e2e_steps * 1e-3) / 1e9
    h2d = h_src.numel() * 2 + h_st.numel() * 4 + h_tt.numel() * 4
    d2h = h_out.numel() * 2
    ok = torch.equal(h_out.view(torch.int16), out.cpu().view(torch.int16))
    e2e = {"value": e2e_val, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps,
           "ms_per_step": e2e_ms / e2e_steps, "matches_device_run": bool(ok),
           "api": "robogoat_b200.host_pipeline.resample_trajectories_host (pinned host in, pinned host out)",
           "pcie_floor_note": "every step moves h2d+d2h bytes over PCIe; that link, not the kernel, bounds this figure"}
    del h_src, h_out

    cpu_baseline = None
    extras = {}
    if rank == 0:
        cpu_baseline = cpu_baseline_leg(world)

    def build_line():
        return {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "arithmetic": "bf16 rows widened to f32, every product and sum rounded separately, one round-to-nearest back to bf16",
            "data": "synthetic",
            "config": {"workload": WORKLOAD,
                       "global_batch": B * world, "parallelism": f"batch-shard x{world}, no collective",
                       "l2": "inputs (1.06 GB) and output (0.52 GB) exceed the 126 MB L2; no flush needed",
                       "bytes_per_step_per_gpu": step_bytes, "bytes_convention": BYTES_CONVENTION,
                       "nccl_nvls": os.environ.get("NCCL_NVLS_ENABLE", "default") if world > 1 else "n/a"},
            "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e, "gpu_launches": args.steps, "clocks": clocks,
            "extras": dict(extras),
        }

    # The side measurements below include collectives.  Should one of them ever stall on some rank, the headline line
    # must still come out: a timer prints it with whatever extras exist and ends the process on every rank.
    guard = LineGuard(rank == 0, build_line, extras, EXTRAS_LIMIT_S if (world > 1 and not args.no_extras) else None)
    guard.start()
    if not args.no_extras:
        try:
            run_extras(L, dev, local, rank, world, peak, extras)
        except Exception as e:  # the headline line must survive a failing side measurement
            extras["error"] = repr(e)
    barrier(world)
    guard.finish()
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


def cpu_baseline_leg(world: int):
    """Oracle port on the host cores, bounded sample (rank 0, N=1 only)."""
    if world != 1:
        return None
    import oracle
    from robogoat_b200 import workloads
    threads = host_threads()
    B_s = 512
    src, st, tt = workloads.resample_inputs(B=B_s, dtype=torch.bfloat16, irregular_targets=True, seed=0,
                                            S=HEADLINE["S"], D=HEADLINE["D"], T=HEADLINE["T"])
    left, right, _ = oracle.brackets(st, tt)
    nbytes = min(workloads.resample_bytes(B_s, HEADLINE["S"], HEADLINE["T"], HEADLINE["D"], 2),
                 workloads.resample_touched_bytes(left, right, HEADLINE["S"], HEADLINE["D"], 2))
    oracle.resample_trajectories(src, st, tt, threads=threads)
    reps, t0 = 0, time.perf_counter()
    while time.perf_counter() - t0 < 10.0 and reps < 200:
        oracle.resample_trajectories(src, st, tt, threads=threads)
        reps += 1
    dt = (time.perf_counter() - t0) / reps
    return {"value": nbytes / dt / 1e9, "unit": UNIT, "cores": threads, "kind": "port",
            "sample": f"B={B_s} rows of the headline batch, {reps} passes (~10 s), oracle port with OpenMP over rows",
            "host_cores": os.cpu_count()}


def run_extras(L, dev, local, rank, world, peak, ex):
    """Fusion and voxelisation figures for the other headline configurations (device-resident inputs), added to ``ex``
    as they are measured."""
    from robogoat_b200 import _lib, ops, workloads
    import robocache
    flush = L2Flush(dev)

    # the headline workload generated from other seeds: how much the figure depends on the draw
    if world == 1:
        per_seed = {}
        for seed in (1, 2, 3, 4):
            s_src, s_st, s_tt = workloads.resample_inputs(B=HEADLINE["B"], S=HEADLINE["S"], D=HEADLINE["D"], T=HEADLINE["T"],
                                                          dtype=torch.bfloat16, irregular_targets=True, seed=seed, device=dev)
            fs = lambda: ops.resample_trajectories_cuda(s_src, s_st, s_tt)
            for _ in range(5):
                r = fs(); del r
            a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a0.record()
            for _ in range(20):
                r = fs(); del r
            a1.record(); torch.cuda.synchronize()
            per_seed[seed] = a0.elapsed_time(a1) / 20
            del s_src, s_st, s_tt
        ex["resample_bf16_B4096_other_seeds_ms"] = {"ms_per_call": per_seed,
                                                   "timing": "20 back-to-back calls through the Python binding (output allocation included)"}

    # fusion throughput, B=16384 per GPU, bf16
    Bf = 16384
    a = workloads.fusion_inputs(B=Bf, dtype=torch.bfloat16, seed=rank, device=dev)
    fb = workloads.fusion_bytes(Bf, 50, 2)
    f = lambda: ops.fuse_multimodal_cuda(*a)
    for _ in range(5):
        f()
    barrier(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    iters = 50
    e0.record()
    for _ in range(iters):
        f()
    e1.record(); torch.cuda.synchronize()
    ms = max_over_ranks(e0.elapsed_time(e1) / iters, world, dev)
    ex["fusion_bf16_B16384"] = {"ms": ms, "GB/s": fb * world / (ms * 1e-3) / 1e9, "frac_of_hbm_peak": fb / (ms * 1e-3) / 1e9 / peak,
                                "bytes_per_gpu": fb, "timing": "50 back-to-back calls incl. output allocation, inputs 0.8 GB > L2"}
    del a
    # fusion latency, B=4
    a4 = workloads.fusion_inputs(B=4, dtype=torch.bfloat16, seed=rank, device=dev)
    med, mean = time_cold(lambda: ops.fuse_multimodal_cuda(*a4), 200, 20, flush)
    ex["fusion_bf16_B4_latency_us"] = {"median": med * 1e3, "mean": mean * 1e3, "timing": "per-call events, L2 flushed before each call"}
    from robogoat_b200.graphs import GraphedOp
    gop = GraphedOp(ops.fuse_multimodal_cuda, a4)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(1000):
        gop.replay()                      # inputs already live in the graph's static buffers
    torch.cuda.synchronize()
    graph_us = (time.perf_counter() - t0) / 1000 * 1e6
    t0 = time.perf_counter()
    for _ in range(1000):
        ops.fuse_multimodal_cuda(*a4)
    torch.cuda.synchronize()
    eager_us = (time.perf_counter() - t0) / 1000 * 1e6
    ex["fusion_bf16_B4_wall_us_per_call"] = {"cuda_graph_replay": graph_us, "direct_call": eager_us,
                                             "timing": "host wall clock over 1000 back-to-back calls (warm L2): what a caller in a loop sees"}

    # voxel occupancy, 500k points, 128^3 (public API: int32 grid; harness format: uint8 grid)
    pts = workloads.voxel_uniform_inputs(500_000, seed=rank, device=dev)
    kw = workloads.VOXEL_OCCUPANCY_GEOMETRY
    med, mean = time_cold(lambda: robocache.voxelize_pointcloud(pts, mode="occupancy", **kw), 200, 20, flush)
    ex["voxel_occupancy_500k_128"] = {"median_us": med * 1e3, "Gpts/s": 500_000 / (med * 1e-3) / 1e9,
                                      "timing": "per-call events incl. grid allocation and zero-fill, L2 flushed before each call"}
    med, mean = time_cold(lambda: ops.voxelize_pointcloud_cuda(pts, None, kw["grid_min"], kw["voxel_size"], kw["grid_size"],
                                                               "occupancy", occupancy_dtype=torch.uint8), 200, 20, flush)
    ex["voxel_occupancy_u8_500k_128"] = {"median_us": med * 1e3, "Gpts/s": 500_000 / (med * 1e-3) / 1e9,
                                         "timing": "same, uint8 occupancy plane (2 MiB zero-fill instead of 8 MiB)"}
    del pts

    # voxel count + mean at scale: N = 2^26 points per GPU, 512^3, F=4
    N = 1 << 26
    pts, feats = workloads.voxel_mixture_inputs(N, seed=rank, device=dev)
    kw = workloads.VOXEL_MIXTURE_GEOMETRY
    for mode in ("count", "mean"):
        fn = (lambda: robocache.voxelize_pointcloud(pts, feats if mode == "mean" else None, mode=mode, **kw))
        for _ in range(3):
            r = fn(); del r
        barrier(world)
        iters = 10
        e0.record()
        for _ in range(iters):
            r = fn(); del r
        e1.record(); torch.cuda.synchronize()
        ms = max_over_ranks(e0.elapsed_time(e1) / iters, world, dev)
        ex[f"voxel_{mode}_64M_512"] = {"ms": ms, "Gpts/s_per_gpu": N / (ms * 1e-3) / 1e9,
                                       "timing": "10 back-to-back calls incl. zero-fill (and normalise for mean); working set > L2"}
    if world > 1:
        from robogoat_b200 import sharding
        # optional gather of the batch-sharded resample outputs (not on the timed headline path)
        shard = torch.empty((HEADLINE["B"], HEADLINE["T"], HEADLINE["D"]), dtype=torch.bfloat16, device=dev)
        for _ in range(2):
            g = sharding.gather_rows(shard, HEADLINE["B"] * world); del g
        barrier(world)
        e0.record()
        for _ in range(3):
            g = sharding.gather_rows(shard, HEADLINE["B"] * world); del g
        e1.record(); torch.cuda.synchronize()
        ms = max_over_ranks(e0.elapsed_time(e1) / 3, world, dev)
        ex["resample_output_all_gather"] = {"ms": ms, "bytes_per_gpu_shard": shard.numel() * 2,
                                            "bus_GB/s": shard.numel() * 2 * (world - 1) / (ms * 1e-3) / 1e9,
                                            "note": "NCCL all-gather of every rank's [4096,250,256] bf16 output into a full copy on every rank"}
        del shard
        fn = lambda: sharding.voxelize_sharded(pts, feats, mode="mean", **kw)
        for _ in range(2):
            r = fn(); del r
        barrier(world)
        e0.record()
        for _ in range(5):
            r = fn(); del r
        e1.record(); torch.cuda.synchronize()
        ms = max_over_ranks(e0.elapsed_time(e1) / 5, world, dev)
        ex["voxel_mean_sharded_with_grid_reduce"] = {"ms": ms, "Gpts/s_total": N * world / (ms * 1e-3) / 1e9,
                                                     "note": "point shards + NCCL all-reduce of the 2.68 GB partial grids + normalise; every rank holds the full grid"}
        fn = lambda: sharding.voxelize_sharded_slab(pts, feats, mode="mean", **kw)
        for _ in range(2):
            r = fn(); del r
        barrier(world)
        e0.record()
        for _ in range(5):
            r = fn(); del r
        e1.record(); torch.cuda.synchronize()
        ms = max_over_ranks(e0.elapsed_time(e1) / 5, world, dev)
        ex["voxel_mean_sharded_slab_output"] = {"ms": ms, "Gpts/s_total": N * world / (ms * 1e-3) / 1e9,
                                                "note": "point shards + NCCL reduce-scatter; each rank keeps the reduced, normalised 1/N slab of z-planes"}
        # point exchange: bucket by owner slab, all-to-all of (id, features) records, scatter into the own slab
        fn = lambda: sharding.voxelize_sharded_exchange(pts, feats, mode="mean", **kw)
        for _ in range(2):
            r = fn(); del r
        barrier(world)
        e0.record()
        for _ in range(5):
            r = fn(); del r
        e1.record(); torch.cuda.synchronize()
        ms = max_over_ranks(e0.elapsed_time(e1) / 5, world, dev)
        K = sharding.sub_parts(512 ** 3, 4, world, "mean")
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        barrier(world)
        ev[0].record()
        ids, fbk, pc = ops.voxel_partition_cuda(pts, feats, kw["grid_min"], kw["voxel_size"], kw["grid_size"], world, K)
        ev[1].record()
        plan = sharding.exchange_plan(sharding._gather_counts(pc), rank, K)
        (ids_in, f_in), _ = sharding.exchange_buckets([ids, fbk], plan["send_counts"], recv_counts=plan["recv_counts"])
        ev[2].record()
        lo_v, hi_v = sharding.slab_bounds(512 ** 3, rank, world)
        r = ops.voxel_scatter_runs_cuda(ids_in.data_ptr(), f_in.data_ptr(), dev, 4, lo_v, hi_v, plan["runs"], K, "mean")
        ev[3].record(); torch.cuda.synchronize()
        stages = [max_over_ranks(ev[i].elapsed_time(ev[i + 1]), world, dev) for i in range(3)]
        received = int(ids_in.numel())
        del r, ids, fbk, ids_in, f_in
        ex["voxel_mean_sharded_point_exchange"] = {
            "ms": ms, "Gpts/s_total": N * world / (ms * 1e-3) / 1e9, "sub_ranges_per_slab": K,
            "stage_ms": {"partition": stages[0], "counts_and_all_to_all": stages[1], "scatter_normalise": stages[2]},
            "points_received_rank0": received,
            "note": "stable partition by owner slab and sub-range + NCCL all-to-all of 20-byte (id, features) records + scatter "
                    "into the rank's own 1/N slab, one L2-sized sub-range per pass; no rank holds a dense grid"}
        # direct form: the partition kernel stores into the owners' buffers over NVLink
        try:
            px = sharding.PointExchange(capacity=int(1.25 * N), feature_width=4)
        except RuntimeError as e:       # raised on every rank alike
            px = None
            ex["voxel_mean_sharded_point_exchange_direct"] = {"unavailable": str(e)[:200]}
        if px is not None:
            fn = lambda: sharding.voxelize_sharded_exchange(pts, feats, mode="mean", direct=px, **kw)
            for _ in range(2):
                r = fn(); del r
            barrier(world)
            e0.record()
            for _ in range(5):
                r = fn(); del r
            e1.record(); torch.cuda.synchronize()
            ms = max_over_ranks(e0.elapsed_time(e1) / 5, world, dev)
            L.rc_set_option(2, 0)                   # sorted chunks written as they lie instead of line-aligned groups
            for _ in range(2):
                r = fn(); del r
            barrier(world)
            e0.record()
            for _ in range(5):
                r = fn(); del r
            e1.record(); torch.cuda.synchronize()
            ms_plain = max_over_ranks(e0.elapsed_time(e1) / 5, world, dev)
            L.rc_set_option(2, 1)
            barrier(world)
            ev[0].record()
            pc, scratch = ops.voxel_partition_count_cuda(pts, kw["grid_min"], kw["voxel_size"], kw["grid_size"], world, K)
            plan = sharding.exchange_plan(sharding._gather_counts(pc), rank, K)
            ev_move = torch.cuda.Event(enable_timing=True)
            ev[1].record()
            fits = max(plan["totals"]) <= px.capacity
            if fits:
                ops.voxel_partition_move_cuda(pts, feats, kw["grid_min"], kw["voxel_size"], kw["grid_size"], world, K,
                                              [px.ids.peers[p // K] for p in range(world * K)],
                                              [px.features.peers[p // K] for p in range(world * K)], plan["dest_start"], scratch,
                                              remote=True)
                ev_move.record()
                px.stream_barrier()
            ev[2].record()
            if fits:
                r = ops.voxel_scatter_runs_cuda(px.ids.ptr, px.features.ptr, dev, 4, lo_v, hi_v, plan["runs"], K, "mean")
                del r
            ev[3].record(); torch.cuda.synchronize()
            stages = [max_over_ranks(ev[i].elapsed_time(ev[i + 1]), world, dev) for i in range(3)]
            sent_remote = sum(c for d, c in enumerate(plan["send_counts"]) if d != rank) * 20
            move_ms = max_over_ranks(ev[1].elapsed_time(ev_move), world, dev) if fits else None
            ex["voxel_mean_sharded_point_exchange_direct"] = {
                "ms": ms, "Gpts/s_total": N * world / (ms * 1e-3) / 1e9, "fits_receive_buffers": fits,
                "ms_without_line_aligned_stores": ms_plain,
                "stage_ms": {"count_and_count_matrix": stages[0], "move_over_nvlink_and_barrier": stages[1], "scatter_normalise": stages[2]},
                "move_kernel_ms": move_ms,
                "nvlink_GB/s_out_per_gpu_during_move": sent_remote / (move_ms * 1e-3) / 1e9 if fits else None,
                "note": "same, but the partition kernel stores its sorted chunks straight into the owners' receive buffers "
                        "(peer memory over NVLink); collectives left: the count matrix and one barrier"}
            px.close()
    else:
        # the two kernels of the point exchange on one GPU: partition for 8 owners, then one owner's bucket into its slab
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        for it in range(3):
            ev[0].record()
            ids, fbk, pc = ops.voxel_partition_cuda(pts, feats, kw["grid_min"], kw["voxel_size"], kw["grid_size"], 8, 4)
            ev[1].record()
            cnts = pc.tolist()                  # host read of the counts: synchronises
            n0 = sum(cnts[:4])
            runs = [(sum(cnts[:k]), cnts[k], k) for k in range(4)]
            ev[2].record()
            r = ops.voxel_scatter_runs_cuda(ids.data_ptr(), fbk.data_ptr(), dev, 4, 0, 512 ** 3 // 8, runs, 4, "mean")
            ev[3].record(); torch.cuda.synchronize()
            part_ms, scat_ms = ev[0].elapsed_time(ev[1]), ev[2].elapsed_time(ev[3])
            del r, ids, fbk
        ex["voxel_point_exchange_kernels_64M_512"] = {
            "partition_8x4_parts_ms": part_ms, "partition_Gpts/s": N / (part_ms * 1e-3) / 1e9,
            "scatter_one_owner_ms": scat_ms, "bucket_points": n0, "scatter_Gpts/s": n0 / (scat_ms * 1e-3) / 1e9,
            "note": "building blocks of the multi-GPU point exchange, timed alone on one GPU"}
    del pts, feats
    pts, feats = workloads.voxel_mixture_inputs(N, seed=rank, device=dev, cluster_sorted=True)
    fn = lambda: robocache.voxelize_pointcloud(pts, feats, mode="mean", **kw)
    for _ in range(3):
        r = fn(); del r
    barrier(world)
    e0.record()
    for _ in range(10):
        r = fn(); del r
    e1.record(); torch.cuda.synchronize()
    ms = max_over_ranks(e0.elapsed_time(e1) / 10, world, dev)
    ex["voxel_mean_64M_512_cluster_sorted"] = {"ms": ms, "Gpts/s_per_gpu": N / (ms * 1e-3) / 1e9,
                                               "timing": "same cloud emitted cluster after cluster (spatially coherent order)"}
    return ex


def run_profile_case(name: str):
    """A few launches of one kernel on a case sized for a profiler capture: larger than L2, well under
    a GB on the device.  Prints one JSON line with the CUDA-event time of the last launch."""
    from robogoat_b200 import ops, workloads
    import robocache
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    if name == "resample":
        src, st, tt = workloads.resample_inputs(B=1024, dtype=torch.bfloat16, irregular_targets=True, seed=0, device=dev,
                                                S=HEADLINE["S"], D=HEADLINE["D"], T=HEADLINE["T"])
        fn = lambda: ops.resample_trajectories_cuda(src, st, tt)
        units = {"B": 1024, "bytes_all_tensors_once": workloads.resample_bytes(1024, 500, 250, 256, 2)}
    elif name == "fusion":
        a = workloads.fusion_inputs(B=4096, dtype=torch.bfloat16, seed=0, device=dev)
        fn = lambda: ops.fuse_multimodal_cuda(*a)
        units = {"B": 4096, "bytes_all_tensors_once": workloads.fusion_bytes(4096, 50, 2)}
    elif name in ("voxel_mean", "voxel_count", "voxel_mean_full"):
        N = (1 << 26) if name.endswith("_full") else (1 << 24)  # the full-size case is for single-pass counter sets only
        pts, feats = workloads.voxel_mixture_inputs(N, seed=0, device=dev)
        kw = workloads.VOXEL_MIXTURE_GEOMETRY
        mode = name.split("_")[1]
        fn = lambda: robocache.voxelize_pointcloud(pts, feats if mode == "mean" else None, mode=mode, **kw)
        units = {"N": N}
    elif name in ("voxel_partition", "voxel_partition_aligned"):
        if name.endswith("_aligned"):       # the write-out used for peer destinations, here with local ones
            from robogoat_b200 import _lib
            _lib.load().rc_set_option(2, 2)
        N = 1 << 24
        pts, feats = workloads.voxel_mixture_inputs(N, seed=0, device=dev)
        kw = workloads.VOXEL_MIXTURE_GEOMETRY
        fn = lambda: ops.voxel_partition_cuda(pts, feats, kw["grid_min"], kw["voxel_size"], kw["grid_size"], 8, 4)
        units = {"N": N, "parts": 32}
    elif name == "voxel_scatter_runs":
        # what one of 2 owners receives from a 2^24-point cloud, cut into 14 L2-sized sub-ranges of its slab
        N = 1 << 24
        pts, feats = workloads.voxel_mixture_inputs(N, seed=0, device=dev)
        kw = workloads.VOXEL_MIXTURE_GEOMETRY
        ids, fbk, pc = ops.voxel_partition_cuda(pts, feats, kw["grid_min"], kw["voxel_size"], kw["grid_size"], 2, 14)
        cnts = pc.tolist()
        runs = [(sum(cnts[:k]), cnts[k], k) for k in range(14)]
        del pts, feats
        fn = lambda: ops.voxel_scatter_runs_cuda(ids.data_ptr(), fbk.data_ptr(), dev, 4, 0, 512 ** 3 // 2, runs, 14, "mean")
        units = {"N": sum(cnts[:14]), "sub_ranges": 14}
    elif name == "voxel_occupancy":
        pts = workloads.voxel_uniform_inputs(500_000, seed=0, device=dev)
        fn = lambda: robocache.voxelize_pointcloud(pts, mode="occupancy", **workloads.VOXEL_OCCUPANCY_GEOMETRY)
        units = {"N": 500_000}
    else:
        raise SystemExit(f"unknown profile case {name}")
    for _ in range(3):
        r = fn(); del r
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record(); r = fn(); ev1.record(); torch.cuda.synchronize()
    print(json.dumps({"profile_case": name, "last_call_ms": ev0.elapsed_time(ev1), **units}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extras", action="store_true")
    ap.add_argument("--profile-case", default=None,
                    help="run 4 launches of one kernel on a small case (resample, fusion, voxel_mean, voxel_count, voxel_occupancy, voxel_partition, voxel_partition_aligned, voxel_scatter_runs; voxel_mean_full = headline size)")
    args = ap.parse_args()
    if args.profile_case:
        run_profile_case(args.profile_case)
        return
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
