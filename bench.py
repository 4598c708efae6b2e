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
TRAFFIC_CAPTURE = os.path.join(ROOT, "profiles", "resample_gather_bf16_B1024.json")   # DRAM bytes of one captured launch
BYTES_CONVENTION = "min(all tensors once, touched rows + times + output)"


# ----------------------------------------------------------------------------- helpers

def captured_traffic(rows: int):
    """DRAM bytes per launch of the resample kernel at ``rows`` batch rows, scaled by rows from the committed profiler
    capture (traffic grows in proportion to the rows); (None, reason) when the capture file is missing."""
    try:
        with open(TRAFFIC_CAPTURE) as f:
            c = json.load(f)
        per_row = (float(c["dram_bytes_read"]) + float(c["dram_bytes_write"])) / float(c["rows_in_capture"])
        return int(per_row * rows), f"ncu dram__bytes_read+write of a B={c['rows_in_capture']} capture, scaled by rows"
    except Exception as e:
        return None, f"no capture file ({type(e).__name__})"


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


class NumaLocal:
    """While active, this process runs on the host cores next to GPU ``index`` (sysfs ``local_cpulist`` of the
    device), so pinned buffers allocated inside land in that socket's memory.  Reads sysfs only; a box without the
    file is left as it is."""

    def __init__(self, index: int):
        self.index, self.old, self.cpus = index, None, None

    def __enter__(self):
        try:
            bus = torch.cuda.get_device_properties(self.index).pci_bus_id
            dom = torch.cuda.get_device_properties(self.index).pci_domain_id
            devid = torch.cuda.get_device_properties(self.index).pci_device_id
            path = f"/sys/bus/pci/devices/{dom:04x}:{bus:02x}:{devid:02x}.0/local_cpulist"
            cpus = set()
            for part in open(path).read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
            allowed = os.sched_getaffinity(0)
            cpus &= allowed
            if cpus and cpus != allowed:
                self.old = allowed
                os.sched_setaffinity(0, cpus)
                self.cpus = len(cpus)
        except Exception:
            self.old = None
        return self

    def __exit__(self, *exc):
        if self.old is not None:
            os.sched_setaffinity(0, self.old)
        return False


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

def headline_config(world: int, step_bytes: int) -> dict:
    """The ``config`` object of the line; both arms print the same keys."""
    B = HEADLINE["B"]
    return {"workload": WORKLOAD, "global_batch": B * world, "parallelism": f"batch-shard x{world}, no collective",
            "l2": "inputs (1.06 GB) and output (0.52 GB) exceed the 126 MB L2; no flush needed",
            "bytes_per_step_per_gpu": step_bytes, "bytes_convention": BYTES_CONVENTION,
            "nccl_nvls": os.environ.get("NCCL_NVLS_ENABLE", "default") if world > 1 else "n/a"}


def run_reference_arm(args):
    """The reference's CPU path for the headline workload on the host cores (rank 0 only): the oracle port with all
    host threads on a bounded sample, timed for at least two seconds, median per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle
    import workloads
    threads = host_threads()
    B_s = 1024                                 # bounded sample: 1/4 of the headline batch per step, 390 MB of rows
    src, st, tt = workloads.resample_inputs(B=B_s, dtype=torch.bfloat16, irregular_targets=True, seed=0,
                                            S=HEADLINE["S"], D=HEADLINE["D"], T=HEADLINE["T"])
    left, right, _ = oracle.brackets(st, tt)
    nbytes = min(workloads.resample_bytes(B_s, HEADLINE["S"], HEADLINE["T"], HEADLINE["D"], 2),
                 workloads.resample_touched_bytes(left, right, HEADLINE["S"], HEADLINE["D"], 2))
    for _ in range(max(args.warmup, 1)):
        oracle.resample_trajectories(src, st, tt, threads=threads)
    # at least K steps and at least two seconds: other ranks' interpreters may still be starting while this runs,
    # and the median over a longer window is not moved by that
    ts, t_begin = [], time.perf_counter()
    while len(ts) < args.steps or (time.perf_counter() - t_begin < 2.0 and len(ts) < 50 * args.steps):
        t0 = time.perf_counter()
        oracle.resample_trajectories(src, st, tt, threads=threads)
        ts.append(time.perf_counter() - t0)
    dt = statistics.median(ts)
    gbs = nbytes / dt / 1e9
    sample = (f"B={B_s} rows per step of the B=4096-per-GPU headline batch (same S, D, T and generator; the CPU rate does not "
              f"depend on B), oracle port, {threads} threads, median of {len(ts)} steps over {time.perf_counter() - t_begin:.1f} s; "
              f"bytes_per_step_per_gpu is the sample's bytes scaled to 4096 rows")
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": headline_config(args.gpus, nbytes * (HEADLINE["B"] // B_s)),
        "cpu_baseline": {"value": gbs, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": gbs, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "steps_timed": len(ts),
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
        import workloads
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
    from robogoat_b200 import _lib, ops
    import workloads
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
                "traffic": captured_traffic(B)[0], "traffic_source": captured_traffic(B)[1], "peak_source": f"of {peak_kind}", "kernel": "interp_gather_kernel<bf16, 16 B, staged, uniform>",
                "kernel_ms": kernel_ms, "bytes_algorithmic_all_tensors_once": algo_bytes,
                "bytes_touched_rows": touched_bytes, "achieved_all_tensors_once": algo_bytes / (kernel_ms * 1e-3) / 1e9}

    # ---- end to end through the public API: pinned host inputs -> device -> op -> pinned host output
    e2e_steps = max(3, min(args.steps, 10))
    with NumaLocal(local) as numa:          # pinned host buffers in the memory of the socket this GPU hangs off
        h_src = torch.empty((B, S, D), dtype=torch.bfloat16).pin_memory()
        h_st, h_tt = torch.empty((B, S), dtype=torch.float32).pin_memory(), torch.empty((B, T), dtype=torch.float32).pin_memory()
        h_out = torch.empty((B, T, D), dtype=torch.bfloat16).pin_memory()
        h_out.zero_()
    h_src.copy_(src); h_st.copy_(st); h_tt.copy_(tt)
    torch.cuda.synchronize()

    from robogoat_b200.host_pipeline import resample_trajectories_host

    def e2e_step():
        # host-buffer entry point of the package: chunked upload / kernel / download on three streams
        resample_trajectories_host(h_src, h_st, h_tt, out=h_out, device=dev, chunk_rows=256)

    e2e_ms, _ = timed_region(e2e_step, e2e_steps, 2, world, dev)
    e2e_val = step_bytes * world / (e2e_ms / e2e_steps * 1e-3) / 1e9
    h2d = h_src.numel() * 2 + h_st.numel() * 4 + h_tt.numel() * 4
    d2h = h_out.numel() * 2
    ok = torch.equal(h_out.view(torch.int16), out.cpu().view(torch.int16))
    # the floor of that figure: the same bytes moved by plain copies and nothing else, upload and download at the
    # same time (the link is full duplex), on all ranks at once
    d_src, d_out = torch.empty_like(src), torch.empty_like(out)
    d_st, d_tt = torch.empty_like(st), torch.empty_like(tt)
    up, down = torch.cuda.Stream(dev), torch.cuda.Stream(dev)

    def copy_step():
        ev = torch.cuda.Event(); ev.record()
        up.wait_event(ev); down.wait_event(ev)
        with torch.cuda.stream(up):
            d_src.copy_(h_src, non_blocking=True); d_st.copy_(h_st, non_blocking=True); d_tt.copy_(h_tt, non_blocking=True)
        with torch.cuda.stream(down):
            h_out.copy_(d_out, non_blocking=True)
        torch.cuda.current_stream().wait_stream(up); torch.cuda.current_stream().wait_stream(down)

    floor_ms, _ = timed_region(copy_step, e2e_steps, 2, world, dev)
    floor_ms /= e2e_steps
    del d_src, d_out, d_st, d_tt
    e2e = {"value": e2e_val, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps,
           "ms_per_step": e2e_ms / e2e_steps, "matches_device_run": bool(ok),
           "api": "robogoat_b200.host_pipeline.resample_trajectories_host (pinned host in, pinned host out)",
           "copy_floor_ms": floor_ms, "frac_of_copy_floor": floor_ms / (e2e_ms / e2e_steps),
           "copy_floor": "one cudaMemcpyAsync per tensor, upload and download on two streams at once, same pinned buffers, "
                         "all ranks at the same time, max over ranks; link GB/s = (h2d + d2h) / copy_floor_ms",
           "copy_floor_link_GB/s": (h2d + d2h) / (floor_ms * 1e-3) / 1e9,
           "pinned_buffers": f"allocated while bound to the {numa.cpus} host cores local to the GPU" if numa.cpus else "allocated without a NUMA binding",
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
            "config": headline_config(world, step_bytes),
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


def cpu_seconds(fn, budget_s: float = 1.5, max_reps: int = 25) -> float:
    """Median wall-clock seconds of ``fn()`` on the host: one warm-up call, then calls until the budget is spent."""
    t0 = time.perf_counter()
    fn()
    first = time.perf_counter() - t0
    if first >= budget_s:            # one call already spends the budget: take it
        return first
    ts, t_end = [], time.perf_counter() + budget_s
    while len(ts) < 2 or (time.perf_counter() < t_end and len(ts) < max_reps):
        t0 = time.perf_counter()
        fn()
        ts.append(time.perf_counter() - t0)
    return statistics.median(ts)


def torch_threads(k: int, fn):
    """Runs ``fn`` with torch's intra-op pool set to ``k`` threads."""
    def run():
        old = torch.get_num_threads()
        torch.set_num_threads(k)
        try:
            return fn()
        finally:
            torch.set_num_threads(old)
    return run


def cpu_records(unit: str, work_per_call: float, scale: float, sample: str, port_fn=None, torch_fn=None,
                port_threaded: bool = True, budget_s: float = 1.5):
    """CPU baselines of one configuration: the C oracle port and the torch restatement of the reference's fallback,
    each with all host threads and with one.  ``work_per_call`` is the sample's work in the unit's numerator
    (bytes for GB/s, points for Gpts/s); ``scale`` = full configuration / sample, used for the ``ms_full_config`` figure."""
    out = []
    threads = host_threads()

    def add(impl, cores, fn):
        try:
            sec = cpu_seconds(fn, budget_s)
        except Exception as e:          # a baseline must never break the line
            out.append({"impl": impl, "cores": cores, "error": repr(e)[:160]})
            return
        out.append({"value": work_per_call / sec / 1e9, "unit": unit, "cores": cores, "kind": "port", "impl": impl,
                    "ms_sample": sec * 1e3, "ms_full_config": sec * scale * 1e3, "sample": sample})

    if port_fn is not None:
        if port_threaded:
            add("C restatement, OpenMP over batch rows", threads, lambda: port_fn(threads))
        add("C restatement, one thread", 1, lambda: port_fn(1))
    if torch_fn is not None:
        add("torch restatement of the reference's Python fallback (oracle/torch_path.py)", threads, torch_threads(threads, torch_fn))
        add("torch restatement, one thread", 1, torch_threads(1, torch_fn))
    return out


def cpu_baseline_leg(world: int):
    """CPU baseline of the headline workload on the host cores, bounded sample (rank 0, N=1 only): the oracle port
    (headline figure) and, under ``also``, the torch restatement of the reference's Python fallback."""
    if world != 1:
        return None
    import oracle
    from oracle import torch_path
    import workloads
    threads = host_threads()
    B_s = 1024                                 # 390 MB working set: larger than the host's last-level cache
    src, st, tt = workloads.resample_inputs(B=B_s, dtype=torch.bfloat16, irregular_targets=True, seed=0,
                                            S=HEADLINE["S"], D=HEADLINE["D"], T=HEADLINE["T"])
    left, right, _ = oracle.brackets(st, tt)
    nbytes = min(workloads.resample_bytes(B_s, HEADLINE["S"], HEADLINE["T"], HEADLINE["D"], 2),
                 workloads.resample_touched_bytes(left, right, HEADLINE["S"], HEADLINE["D"], 2))
    oracle.resample_trajectories(src, st, tt, threads=threads)
    ts, t_end = [], time.perf_counter() + 8.0
    while time.perf_counter() < t_end and len(ts) < 200:
        t0 = time.perf_counter()
        oracle.resample_trajectories(src, st, tt, threads=threads)
        ts.append(time.perf_counter() - t0)
    dt = statistics.median(ts)
    scale = HEADLINE["B"] / 256
    s256 = (src[:256], st[:256], tt[:256])
    also = cpu_records(UNIT, nbytes / 4, scale, "B=256 rows of the headline batch (the fallback loops over rows: linear in B)",
                       port_fn=lambda k: oracle.resample_trajectories(*s256, threads=k),
                       torch_fn=lambda: torch_path.interpolate_stream(*s256), budget_s=2.0)
    return {"value": nbytes / dt / 1e9, "unit": UNIT, "cores": threads, "kind": "port",
            "sample": f"B={B_s} rows of the headline batch ({B_s * 500 * 256 * 2 >> 20} MB of rows), median of {len(ts)} passes (~8 s), "
                      f"oracle port with OpenMP over rows",
            "host_cores": os.cpu_count(), "also": also}


def gpu_record(ms: float, work: float, unit: str, nbytes: int, peak: float, timing: str, world: int = 1) -> dict:
    """One measured configuration: time, rate in the metric's unit (whole job), algorithmic bytes per GPU and the
    fraction of the measured HBM copy peak those bytes amount to."""
    rec = {"ms": ms, "rate": work * world / (ms * 1e-3) / 1e9, "unit": unit, "bytes_algorithmic": int(nbytes),
           "GB/s_per_gpu": nbytes / (ms * 1e-3) / 1e9, "frac_of_hbm_peak": nbytes / (ms * 1e-3) / 1e9 / peak, "timing": timing}
    return rec


def run_extras(L, dev, local, rank, world, peak, ex):
    """The other configurations of the headline benchmark (device-resident inputs), added to ``ex`` as they are
    measured: every record carries ms, rate, algorithmic bytes and their fraction of the HBM peak, and — on one GPU —
    the CPU baselines of that configuration (the C oracle port and the torch restatement of the reference's fallback)."""
    from robogoat_b200 import _lib, ops
    import workloads
    import robocache
    flush = L2Flush(dev)
    cpu = (world == 1 and rank == 0)
    if cpu:
        import oracle
        from oracle import torch_path

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

    # configs[0]: fp32 B=32 S=500 D=256 T=250, linspace targets shared by the batch (the reference's own CPU-runnable case)
    c1 = workloads.resample_inputs(B=32, S=500, D=256, T=250, dtype=torch.float32, irregular_targets=False, seed=rank)
    d1 = [t.to(dev) for t in c1]
    b1 = workloads.resample_bytes(32, 500, 250, 256, 4)
    med, mean = time_cold(lambda: robocache.resample_trajectories(*d1), 200, 20, flush)
    ex["cfg1_resample_fp32_B32"] = gpu_record(med, b1, "GB/s", b1, peak, "per-call events through the public API incl. output allocation, L2 flushed before each call (median of 200)", world)
    ex["cfg1_resample_fp32_B32"]["reference_published_h100_ms"] = {"gpu_p50": 2.605, "torch_cpu_p50": 38.385,
                                                                  "source": "robocache/bench/results/benchmark_h100_20251106_172811.csv:4-5 (bf16, wall-clock harness)"}
    if cpu:
        ex["cfg1_resample_fp32_B32"]["cpu_baseline"] = cpu_records(
            "GB/s", b1, 1.0, "the full configuration", port_fn=lambda k: oracle.resample_trajectories(*c1, threads=k),
            torch_fn=lambda: torch_path.interpolate_stream(*c1), budget_s=1.0)
    del d1

    # configs[2]: fusion throughput, B=16384 per GPU, bf16
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
    ex["fusion_bf16_B16384"] = gpu_record(ms, fb, "GB/s", fb, peak, "50 back-to-back calls incl. output allocation, inputs 0.8 GB > L2", world)
    if cpu:
        a256 = [x[:256].cpu() for x in a]
        ex["fusion_bf16_B16384"]["cpu_baseline"] = cpu_records(
            "GB/s", fb / 64, 64.0, "B=256 items of the batch (the fallback loops over items: linear in B)",
            port_fn=lambda k: oracle.fuse_multimodal(*a256, threads=k), torch_fn=lambda: torch_path.fuse_multimodal(*a256))
    del a
    # fusion latency, B=4
    a4 = workloads.fusion_inputs(B=4, dtype=torch.bfloat16, seed=rank, device=dev)
    med, mean = time_cold(lambda: ops.fuse_multimodal_cuda(*a4), 200, 20, flush)
    fb4 = workloads.fusion_bytes(4, 50, 2)
    ex["fusion_bf16_B4"] = gpu_record(med, fb4, "GB/s", fb4, peak, "per-call events, L2 flushed before each call (median of 200); a latency case: "
                                      "434 560 B take 0.07 us at the HBM peak, the call is launch-bound", world)
    ex["fusion_bf16_B4"]["latency_us"] = {"median": med * 1e3, "mean": mean * 1e3}
    if cpu:
        a4c = [x.cpu() for x in a4]
        ex["fusion_bf16_B4"]["cpu_baseline"] = cpu_records(
            "GB/s", fb4, 1.0, "the full configuration", port_fn=lambda k: oracle.fuse_multimodal(*a4c, threads=k),
            torch_fn=lambda: torch_path.fuse_multimodal(*a4c), budget_s=0.5)
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
    ex["fusion_bf16_B4"]["wall_us_per_call"] = {"cuda_graph_replay": graph_us, "direct_call": eager_us,
                                                "timing": "host wall clock over 1000 back-to-back calls (warm L2): what a caller in a loop sees"}

    # configs[3]: voxel occupancy, 500k points, 128^3 (public API: int32 grid; harness format: uint8 grid)
    pts = workloads.voxel_uniform_inputs(500_000, seed=rank, device=dev)
    kw = workloads.VOXEL_OCCUPANCY_GEOMETRY
    med, mean = time_cold(lambda: robocache.voxelize_pointcloud(pts, mode="occupancy", **kw), 200, 20, flush)
    vb = workloads.voxel_bytes(500_000, 0, 128 ** 3, "occupancy")["total"]
    ex["voxel_occupancy_500k_128"] = gpu_record(med, 500_000, "Gpts/s", vb, peak,
                                                "per-call events incl. grid allocation and zero-fill, L2 flushed before each call; "
                                                "14.4 MB take 2.2 us at the HBM peak: launch-bound", world)
    med8, _ = time_cold(lambda: ops.voxelize_pointcloud_cuda(pts, None, kw["grid_min"], kw["voxel_size"], kw["grid_size"],
                                                             "occupancy", occupancy_dtype=torch.uint8), 200, 20, flush)
    ex["voxel_occupancy_u8_500k_128"] = gpu_record(med8, 500_000, "Gpts/s", 6_000_000 + 128 ** 3, peak,
                                                   "same, uint8 occupancy plane (2 MiB zero-fill instead of 8 MiB)", world)
    if cpu:
        pc = pts.cpu()
        ex["voxel_occupancy_500k_128"]["cpu_baseline"] = cpu_records(
            "Gpts/s", 500_000, 1.0, "the full configuration (the torch fallback clamps out-of-grid points and is x-major: a timed baseline, not the oracle)",
            port_fn=lambda k: oracle.voxelize_pointcloud(pc, None, mode="occupancy", **kw), port_threaded=False,
            torch_fn=lambda: torch_path.voxelize_pointcloud(pc, None, mode="occupancy", **kw), budget_s=1.0)
    del pts

    # configs[4]: voxel count + mean at scale: N = 2^26 points per GPU, 512^3, F=4
    N = 1 << 26
    pts, feats = workloads.voxel_mixture_inputs(N, seed=rank, device=dev)
    kw = workloads.VOXEL_MIXTURE_GEOMETRY
    occupied = int((robocache.voxelize_pointcloud(pts, mode="count", **kw) > 0).sum().item())
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
        vb = workloads.voxel_bytes(N, 4, 512 ** 3, mode, occupied)["total"]
        ex[f"voxel_{mode}_64M_512"] = gpu_record(ms, N, "Gpts/s", vb, peak,
                                                 "10 back-to-back calls incl. zero-fill (and normalise for mean); working set > L2", world)
        ex[f"voxel_{mode}_64M_512"]["Gpts/s_per_gpu"] = N / (ms * 1e-3) / 1e9
        ex[f"voxel_{mode}_64M_512"]["occupied_voxels"] = occupied
        if cpu:
            Ns = 1 << 22
            ps, fs_ = pts[:Ns].cpu(), feats[:Ns].cpu()
            ex[f"voxel_{mode}_64M_512"]["cpu_baseline"] = cpu_records(
                "Gpts/s", Ns, N / Ns, "the first 2^22 points of the cloud into the same 512^3 grid, scaled linearly in N",
                port_fn=lambda k: oracle.voxelize_pointcloud(ps, fs_ if mode == "mean" else None, mode=mode, **kw), port_threaded=False,
                torch_fn=lambda: torch_path.voxelize_pointcloud(ps, fs_ if mode == "mean" else None, mode=mode, **kw), budget_s=2.0)
    if world > 1:
        multi_gpu_extras(L, dev, rank, world, ex, pts, feats, kw, N,
                         {m: ex[f"voxel_{m}_64M_512"]["ms"] for m in ("count", "mean")})
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
    del pts, feats
    if world == 1:
        # the older batched surface: 8 clouds of 500 k points -> float density [8,128,128,128] in one launch, and a
        # truncated signed distance grid from 4 x 65536 surface points (unit sphere, normals outwards)
        from robogoat_b200 import batched
        okw = workloads.VOXEL_OCCUPANCY_GEOMETRY
        bp = torch.stack([workloads.voxel_uniform_inputs(500_000, seed=10 + b) for b in range(8)]).to(dev)
        origin, dhw = okw["grid_min"], list(reversed(okw["grid_size"]))
        fn = lambda: batched.voxelize_density_batched(bp, dhw, okw["voxel_size"], origin)
        med, _ = time_cold(fn, 20, 5, flush)
        nb = bp.numel() * 4 + 2 * 8 * 128 ** 3 * 4
        ex["voxel_density_batched_8x500k_128"] = gpu_record(med, 8 * 500_000, "Gpts/s", nb, peak,
                                                            "median of 20 cold-L2 calls; one launch for the batch, zero-fill included")
        g = torch.Generator().manual_seed(5)
        sp = torch.randn(4, 65536, 3, generator=g)
        sp = sp / sp.norm(dim=2, keepdim=True)
        spd, nrm = (sp * 2.0).to(dev), sp.to(dev)
        fn = lambda: batched.voxelize_tsdf(spd, nrm, [128, 128, 128], 0.05, [-3.2, -3.2, -3.2], 0.15)
        med, _ = time_cold(fn, 20, 5, flush)
        _, w = fn()
        pairs = float(w.sum())
        ex["voxel_tsdf_4x65536_128"] = {"ms": med, "point_voxel_updates": pairs, "G_updates/s": pairs / (med * 1e-3) / 1e9,
                                        "timing": "median of 20 cold-L2 calls; truncation 3 voxels; clears and decode pass included"}
    return ex


def sharded_parity(dev, rank, world, px, bx=None, bxs=None) -> dict:
    """Every sharded voxel form on a cloud small enough for the CPU oracle (2^20 mixture points into 128^3), checked
    on every rank against the oracle run on the whole cloud: occupancy and counts exact, means within the oracle's
    tolerance.  Returns one flag per form, true only if it held on all ranks."""
    import oracle
    import workloads
    from robogoat_b200 import sharding
    import torch.distributed as dist
    n = 1 << 20
    p_h, f_h = workloads.voxel_mixture_inputs(n, seed=99)
    p_h = p_h * 0.25
    kw = dict(grid_min=[-6.4, -6.4, -6.4], voxel_size=0.1, grid_size=[128, 128, 128])
    V = 128 ** 3
    occ = oracle.voxelize_pointcloud(p_h, None, mode="occupancy", **kw).reshape(V)
    cnt = oracle.voxelize_pointcloud(p_h, None, mode="count", **kw).reshape(V)
    mean, mcnt, sabs = oracle.voxelize_pointcloud(p_h, f_h, mode="mean", return_aux=True, **kw)
    tol = oracle.mean_tolerance(mcnt, sabs, mean).reshape(V, 4)
    mean = mean.reshape(V, 4)
    lo, hi = sharding.shard_bounds(n, rank, world)
    pl, fl = p_h[lo:hi].to(dev), f_h[lo:hi].to(dev)

    def count_ok(got, a=0, b=V):
        return bool(torch.equal(got.reshape(-1).cpu(), cnt[a:b]))

    def mean_ok(got, a=0, b=V):
        return bool(((got.reshape(-1, 4).cpu() - mean[a:b]).abs() <= tol[a:b]).all())

    sa, sb = rank * V // world, (rank + 1) * V // world       # reduce-scatter slabs
    xa, xb = sharding.slab_bounds(V, rank, world)             # point-exchange slabs
    flags = {}
    flags["all_reduce"] = (bool(torch.equal(sharding.voxelize_sharded(pl, None, mode="occupancy", **kw).reshape(V).cpu(), occ))
                           and count_ok(sharding.voxelize_sharded(pl, None, mode="count", **kw))
                           and mean_ok(sharding.voxelize_sharded(pl, fl, mode="mean", **kw)))
    flags["slab"] = (count_ok(sharding.voxelize_sharded_slab(pl, None, mode="count", **kw), sa, sb)
                     and mean_ok(sharding.voxelize_sharded_slab(pl, fl, mode="mean", **kw), sa, sb))
    flags["exchange"] = (count_ok(sharding.voxelize_sharded_exchange(pl, None, mode="count", **kw), xa, xb)
                         and mean_ok(sharding.voxelize_sharded_exchange(pl, fl, mode="mean", **kw), xa, xb))
    if px is not None:
        flags["exchange_direct"] = (count_ok(sharding.voxelize_sharded_exchange(pl, None, mode="count", direct=px, **kw), xa, xb)
                                    and mean_ok(sharding.voxelize_sharded_exchange(pl, fl, mode="mean", direct=px, **kw), xa, xb))
        flags["exchange_direct_batched"] = (
            count_ok(sharding.voxelize_sharded_exchange(pl, None, mode="count", direct=px, batches=4, **kw), xa, xb)
            and mean_ok(sharding.voxelize_sharded_exchange(pl, fl, mode="mean", direct=px, batches=4, **kw), xa, xb))
    for key, ex_ in (("bucket_exchange", bx), ("bucket_exchange_store", bxs)):
        if ex_ is None:
            continue
        flags[key] = True
        for _ in range(2):          # twice: the second call's records meet pools that have just been read
            got, gcnt = sharding.voxelize_sharded_buckets(pl, fl, ex_, return_counts=True, slices=1, **kw)
            flags[key] = flags[key] and count_ok(gcnt, xa, xb) and mean_ok(got, xa, xb)
        if not ex_.fetch:
            # sliced form, on pools sized for this cloud so that every slice carries points
            small = sharding.BucketExchange(points_per_rank=(n + world - 1) // world + 3000, n_voxels=V)
            flags[key + "_sliced"] = True
            for slices in (4, 4, 3):
                got, gcnt = sharding.voxelize_sharded_buckets(pl, fl, small, return_counts=True, slices=slices, **kw)
                flags[key + "_sliced"] = flags[key + "_sliced"] and count_ok(gcnt, xa, xb) and mean_ok(got, xa, xb)
            small.close()
    sr = None
    try:
        sr = sharding.SparseReduce(records_per_pair=V // world + 4096)
    except RuntimeError:
        pass
    if sr is not None:
        flags["sparse_reduce"] = True
        for _ in range(2):
            got, gcnt = sharding.voxelize_sharded_sparse(pl, fl, sr, return_counts=True, **kw)
            flags["sparse_reduce"] = flags["sparse_reduce"] and count_ok(gcnt, xa, xb) and mean_ok(got, xa, xb)
            flags["sparse_reduce"] = flags["sparse_reduce"] and count_ok(sharding.voxelize_sharded_sparse(pl, None, sr, mode="count", **kw), xa, xb)
        sr.close()
    sg = None
    try:
        sg = sharding.SparseGather(records_per_rank=V)
    except RuntimeError:
        pass
    if sg is not None:
        ok = True
        for _ in range(2):
            ok = ok and bool(torch.equal(sharding.voxelize_sharded_sparse_full(pl, None, sg, mode="occupancy", **kw).reshape(V).cpu(), occ))
            ok = ok and count_ok(sharding.voxelize_sharded_sparse_full(pl, None, sg, mode="count", **kw))
            ok = ok and mean_ok(sharding.voxelize_sharded_sparse_full(pl, fl, sg, mode="mean", **kw))
        flags["sparse_all_gather"] = ok
        sg.close()
    names = sorted(flags)
    t = torch.tensor([1 if flags[k] else 0 for k in names], dtype=torch.int32, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    return {k: bool(v) for k, v in zip(names, t.tolist())}


def multi_gpu_extras(L, dev, rank, world, ex, pts, feats, kw, N, single_ms):
    """Voxelisation over point shards (2^26 points per GPU into 512^3), every form timed in count and mean mode and
    checked against the oracle on a small cloud first; occupancy at the 500 k / 128^3 configuration with the
    reference's all_reduce(MAX).  ``efficiency`` = one GPU's time for its 2^26 points / this time (weak scaling)."""
    from robogoat_b200 import sharding, ops
    import workloads
    import torch.distributed as dist
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def timed(fn, iters=5, warm=2):
        for _ in range(warm):
            r = fn(); del r
        barrier(world)
        e0.record()
        for _ in range(iters):
            r = fn(); del r
        e1.record(); torch.cuda.synchronize()
        return max_over_ranks(e0.elapsed_time(e1) / iters, world, dev)

    # optional gather of the batch-sharded resample outputs (not on the timed headline path)
    shard = torch.empty((HEADLINE["B"], HEADLINE["T"], HEADLINE["D"]), dtype=torch.bfloat16, device=dev)
    ms = timed(lambda: sharding.gather_rows(shard, HEADLINE["B"] * world), 3)
    ex["resample_output_all_gather"] = {"ms": ms, "bytes_per_gpu_shard": shard.numel() * 2,
                                        "bus_GB/s": shard.numel() * 2 * (world - 1) / (ms * 1e-3) / 1e9,
                                        "note": "NCCL all-gather of every rank's [4096,250,256] bf16 output into a full copy on every rank"}
    del shard

    try:
        px = sharding.PointExchange(capacity=int(1.25 * N), feature_width=4)
    except RuntimeError as e:       # raised on every rank alike
        px = None
        ex["voxel_sharded_direct_unavailable"] = str(e)[:200]
    bx = bxs = None         # bxs: the fetching transport (measured slower; not timed by default)
    try:
        bx = sharding.BucketExchange(points_per_rank=N, n_voxels=512 ** 3)
    except RuntimeError as e:
        ex["voxel_sharded_bucket_exchange_unavailable"] = str(e)[:200]
    parity = sharded_parity(dev, rank, world, px, bx, bxs)
    ex["voxel_sharded_parity"] = {"parity": parity,
                                  "checked": "2^20 mixture points into 128^3 on every rank against the CPU oracle run on the whole cloud: "
                                             "occupancy and counts exact, means within 1e-5 relative + 1e-6 of the mean summand"}

    # configs[3] over point shards: 500 000 points in all, private uint8 planes, all_reduce(MAX) as the reference's
    # multi-GPU test does (robocache/tests/test_multi_gpu.py:60-81)
    okw = workloads.VOXEL_OCCUPANCY_GEOMETRY
    allp = workloads.voxel_uniform_inputs(500_000, seed=0, device=dev)
    lo, hi = sharding.shard_bounds(500_000, rank, world)
    mine = allp[lo:hi].contiguous()
    ms = timed(lambda: sharding.voxelize_sharded(mine, None, mode="occupancy", **okw), 50, 10)
    ex["voxel_occupancy_500k_128_sharded_max_reduce"] = {
        "ms": ms, "Gpts/s_total": (500_000 / (ms * 1e-3) / 1e9) if parity.get("all_reduce") else 0.0, "parity": parity.get("all_reduce"),
        "note": "500 000 points split over the ranks, private uint8 occupancy planes, NCCL all_reduce(MAX) of 2 MiB, int32 result on every rank; "
                "50 back-to-back calls (warm L2): the collective's latency bounds it"}
    try:
        sg_small = sharding.SparseGather(records_per_rank=1 << 18)
        ms = timed(lambda: sharding.voxelize_sharded_sparse_full(mine, None, sg_small, mode="occupancy", check=False, **okw), 50, 10)
        bad = sg_small.failed()
        ex["voxel_occupancy_500k_128_sharded_sparse_all_gather"] = {
            "ms": ms, "Gpts/s_total": (500_000 / (ms * 1e-3) / 1e9) if (parity.get("sparse_all_gather") and not bad) else 0.0,
            "parity": bool(parity.get("sparse_all_gather")) and not bad,
            "note": "same result (int32 occupancy grid on every rank) without NCCL: every rank lists its occupied voxels in its own memory, "
                    "a flag barrier over NVLink, every rank merges the others' lists read over NVLink; 50 back-to-back calls (warm L2)"}
        sg_small.close()
    except RuntimeError as e:
        ex["voxel_sharded_sparse_all_gather_unavailable"] = str(e)[:200]
    del allp, mine

    forms = [("all_reduce", "all_reduce", lambda m: sharding.voxelize_sharded(pts, feats if m == "mean" else None, mode=m, **kw),
              "point shards + NCCL all-reduce of the dense partial grids (+ normalise); every rank holds the full grid"),
             ("reduce_scatter_slab", "slab", lambda m: sharding.voxelize_sharded_slab(pts, feats if m == "mean" else None, mode=m, **kw),
              "point shards + NCCL reduce-scatter; each rank keeps the reduced (normalised) 1/N slab of z-planes"),
             ("point_exchange", "exchange", lambda m: sharding.voxelize_sharded_exchange(pts, feats if m == "mean" else None, mode=m, **kw),
              "stable partition by owner slab and sub-range + NCCL all-to-all of (id, features) records + scatter into the own slab")]
    if px is not None:
        forms += [("point_exchange_direct", "exchange_direct",
                   lambda m: sharding.voxelize_sharded_exchange(pts, feats if m == "mean" else None, mode=m, direct=px, **kw),
                   "the partition kernel stores its sorted chunks straight into the owners' receive buffers (peer memory over NVLink)"),
                  ("point_exchange_direct_batched", "exchange_direct_batched",
                   lambda m: sharding.voxelize_sharded_exchange(pts, feats if m == "mean" else None, mode=m, direct=px, batches=4, **kw),
                   "same in four slices of the local cloud: the stores of slice i+1 overlap the owners' accumulation of slice i")]
    if bx is not None:
        forms.append(("bucket_exchange", "bucket_exchange", lambda m: sharding.voxelize_sharded_buckets(pts, feats, bx, slices=1, **kw),
                      "one bucket kernel sorts every chunk by (owner, sub-range) and stores each owner's records into a fixed block of "
                      "that owner's pool over NVLink; no counts, no host synchronisation, two barriers on the stream; mean mode only"))
        forms.append(("bucket_exchange_sliced", "bucket_exchange_sliced",
                      lambda m: sharding.voxelize_sharded_buckets(pts, feats, bx, slices=4, **kw),
                      "the same in four slices on three streams: while slice s+1 is bucketed and stored over NVLink (a grid of 2 CTAs "
                      "per SM: the stores are link-bound), the owners accumulate slice s; per-slice barriers on a stream of their own"))
    sr = None
    try:
        sr = sharding.SparseReduce(records_per_pair=(12 << 20) // world)
    except RuntimeError as e:
        ex["voxel_sharded_sparse_reduce_unavailable"] = str(e)[:200]
    if sr is not None:
        forms.append(("sparse_reduce", "sparse_reduce",
                      lambda m: sharding.voxelize_sharded_sparse(pts, feats if m == "mean" else None, sr, check=False, mode=m, **kw),
                      "every rank bins its own points into a private full grid, then only the occupied voxels of the other ranks' slabs "
                      "travel (24 B per occupied voxel instead of 20 B per point) and the owners add them to their own slab; pays "
                      "because this cloud puts 13 points into an occupied voxel on average - data dependent, unlike the exchanges"))
    sg = None
    try:
        sg = sharding.SparseGather(records_per_rank=12 << 20)
    except RuntimeError as e:
        ex["voxel_sharded_sparse_all_gather_unavailable"] = str(e)[:200]
    if sg is not None:
        forms.append(("sparse_all_gather", "sparse_all_gather",
                      lambda m: sharding.voxelize_sharded_sparse_full(pts, feats if m == "mean" else None, sg, mode=m, check=False, **kw),
                      "the full grid on every rank, like the all-reduce form: private full grids, every rank lists its occupied voxels in "
                      "its own memory and merges the other ranks' lists read over NVLink; data dependent like the sparse reduction"))
    if bxs is not None:
        forms.append(("bucket_exchange_fetch", "bucket_exchange_store", lambda m: sharding.voxelize_sharded_buckets(pts, feats, bxs, **kw),
                      "same pools in the sources' own memory; every owner's accumulation kernel fetches its blocks over NVLink as it goes"))
    for mode in ("mean", "count"):
        for name, pkey, fn, note in forms:
            if name.startswith("bucket_exchange") and mode != "mean":
                continue
            ms = timed(lambda: fn(mode))
            ok = bool(parity.get(pkey))
            ex[f"voxel_{mode}_sharded_{name}"] = {"ms": ms, "Gpts/s_total": (N * world / (ms * 1e-3) / 1e9) if ok else 0.0, "parity": ok,
                                                  "efficiency": single_ms[mode] / ms, "single_gpu_ms": single_ms[mode], "note": note}

    # stages of the all-to-all and of the direct form (mean mode), each max over ranks
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
    ex["voxel_mean_sharded_point_exchange"].update({
        "sub_ranges_per_slab": K, "points_received_rank0": int(ids_in.numel()),
        "stage_ms": {"partition": stages[0], "counts_and_all_to_all": stages[1], "scatter_normalise": stages[2]}})
    del r, ids, fbk, ids_in, f_in
    if px is not None:
        L.rc_set_option(2, 0)                   # sorted chunks written as they lie instead of line-aligned groups
        ms_plain = timed(lambda: sharding.voxelize_sharded_exchange(pts, feats, mode="mean", direct=px, **kw))
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
        ex["voxel_mean_sharded_point_exchange_direct"].update({
            "fits_receive_buffers": fits, "ms_without_line_aligned_stores": ms_plain,
            "stage_ms": {"count_and_count_matrix": stages[0], "move_over_nvlink_and_barrier": stages[1], "scatter_normalise": stages[2]},
            "move_kernel_ms": move_ms,
            "nvlink_GB/s_out_per_gpu_during_move": sent_remote / (move_ms * 1e-3) / 1e9 if fits else None,
            "bound": "the move kernel (NVLink, measured 770 GB/s per direction) and the owner's atomics run back to back here; "
                     "the batched form overlaps them"})
        px.close()
    if sg is not None:
        bad = sg.failed()
        for m_ in ("mean", "count"):
            ex[f"voxel_{m_}_sharded_sparse_all_gather"]["record_lists_overflowed_or_barrier_timed_out"] = bad
            if bad:
                ex[f"voxel_{m_}_sharded_sparse_all_gather"].update({"Gpts/s_total": 0.0, "parity": False})
        sg.close()
    if sr is not None and bx is not None:
        # full size, where no CPU oracle is affordable: the two fastest forms share no kernel after the points are read
        # (sorted records over NVLink against private grids + occupied voxels), so their slabs must agree - counts
        # exactly, means to rounding - and the counts of all slabs must add up to the points inside the grid
        g1, c1 = sharding.voxelize_sharded_buckets(pts, feats, bx, return_counts=True, slices=4, **kw)
        g2, c2 = sharding.voxelize_sharded_sparse(pts, feats, sr, return_counts=True, check=False, **kw)
        same_counts = bool(torch.equal(c1, c2))
        worst = float(((g1 - g2).abs() - 1e-5 * g1.abs()).max().item()) if g1.numel() else 0.0
        inside = torch.tensor([int(c2.sum(dtype=torch.int64).item()), int(c1.sum(dtype=torch.int64).item())], dtype=torch.int64, device=dev)
        dist.all_reduce(inside)
        cgrid = sharding.voxelize_sharded_slab(pts, None, mode="count", **kw)
        total = torch.tensor([int(cgrid.sum(dtype=torch.int64).item())], dtype=torch.int64, device=dev)
        dist.all_reduce(total)
        okf = torch.tensor([1 if (same_counts and worst <= 1e-5) else 0], dtype=torch.int32, device=dev)
        dist.all_reduce(okf, op=dist.ReduceOp.MIN)
        ex["voxel_mean_sharded_full_scale_agreement"] = {
            "bucket_exchange_sliced_vs_sparse_reduce": bool(okf.item()) and inside[0].item() == inside[1].item() == total[0].item(),
            "points_inside_grid_all_ranks": int(total[0].item()), "counted_by_sparse_reduce": int(inside[0].item()),
            "counted_by_bucket_exchange": int(inside[1].item()),
            "checked": "per rank: slab counts identical, |mean difference| <= 1e-5 (1 + |mean|); over all ranks: counts add up to the "
                       "reduce-scatter count grid's total"}
        del g1, c1, g2, c2, cgrid
    if sr is not None:
        rec = ex["voxel_mean_sharded_sparse_reduce"]
        overflowed = sr.failed()                # any record list overflowed on any rank since the parity check
        rec["record_lists_overflowed"] = overflowed
        if overflowed:              # the same occupied voxels travel in both modes
            for m_ in ("mean", "count"):
                ex[f"voxel_{m_}_sharded_sparse_reduce"].update({"Gpts/s_total": 0.0, "parity": False})
        # stages, each max over ranks
        Vv = 512 ** 3
        a_v, b_v = sharding.slab_bounds(Vv, rank, world)
        others = [(rank + k) % world for k in range(1, world)]
        d_ids, d_sums, d_counts, d_nrec = sr.destinations(others)
        s_ids, s_sums, s_counts, s_nrec = sr.sources(others)
        barrier(world)
        sr.stream_barrier()
        ev[0].record()
        g_, c_ = ops.voxelize_pointcloud_cuda(pts, feats, kw["grid_min"], kw["voxel_size"], kw["grid_size"], "mean", normalize=False)
        g_, c_ = g_.view(Vv, 4), c_.view(Vv)
        ev[1].record()
        ops.voxel_sparse_send_cuda(g_, c_, [sharding.slab_bounds(Vv, d, world) for d in others], sr.capacity, d_ids, d_sums, d_counts,
                                   d_nrec, sr.cursors, sr.overflow)
        ev[2].record()
        sr.stream_barrier()
        ops.voxel_sparse_merge_cuda(s_ids, s_sums, s_counts, s_nrec, sr.capacity, g_, c_, a_v, b_v)
        ev[3].record(); torch.cuda.synchronize()
        sent = int(sr.cursors[:len(others)].sum().item())
        stages = [max_over_ranks(ev[i].elapsed_time(ev[i + 1]), world, dev) for i in range(3)]
        rec.update({"stage_ms": {"private_full_grid": stages[0], "send_occupied_voxels": stages[1], "barrier_merge_normalise": stages[2]},
                    "records_sent_rank0": sent, "bytes_sent_rank0": sent * 24, "capacity_per_pair": sr.capacity,
                    "nvlink_GB/s_out_during_send": sent * 24 / (stages[1] * 1e-3) / 1e9})
        del g_, c_
        sr.close()
    for key, ex_ in (("bucket_exchange", bx), ("bucket_exchange_fetch", bxs)):
        if ex_ is None:
            continue
        # stages of the bucket forms, each max over ranks
        a_v, b_v = sharding.slab_bounds(512 ** 3, rank, world)
        d_ids, d_feats, d_runs, first_block, pool_blocks = ex_.destinations()
        s_ids, s_feats, s_runs, per_source = ex_.sources()
        barrier(world)
        ex_.stream_barrier()
        ev[0].record()
        ops.voxel_bucket_exchange_cuda(pts, feats, kw["grid_min"], kw["voxel_size"], kw["grid_size"], world, ex_.per_group, ex_.chunks,
                                       first_block, pool_blocks, d_ids, d_feats, d_runs)
        ev[1].record()
        ex_.stream_barrier()
        ev[2].record()
        r = ops.voxel_scatter_buckets_cuda(s_ids, s_feats, s_runs, per_source, ex_.per_group, dev, a_v, b_v)
        ev[3].record(); torch.cuda.synchronize()
        stages = [max_over_ranks(ev[i].elapsed_time(ev[i + 1]), world, dev) for i in range(3)]
        del r
        L.rc_set_option(5, 0)                   # the bucket kernel's write-out by ordinary stores instead of bulk copies
        ms_plain = timed(lambda: sharding.voxelize_sharded_buckets(pts, feats, ex_, slices=1, **kw))
        L.rc_set_option(5, 1)
        ex[f"voxel_mean_sharded_{key}"]["ms_with_ordinary_stores"] = ms_plain
        remote_bytes = N * 20 * (world - 1) / world
        link_stage = stages[2] if ex_.fetch else stages[0]
        ex[f"voxel_mean_sharded_{key}"].update({
            "sub_ranges_per_slab": ex_.per_group,
            "stage_ms": {"bucket_kernel": stages[0], "barrier": stages[1], "clear_accumulate_normalise": stages[2]},
            "nvlink_GB/s_per_gpu_during_the_stage_that_crosses_it": remote_bytes / (link_stage * 1e-3) / 1e9,
            "bound": "bucket kernel: its own work (0.65 ms on one GPU) and, when it stores remotely, the record bytes that must cross NVLink / "
                     "770 GB/s per direction; accumulation: the rate at which L2 retires atomics and, when it fetches, the same link bound"})
        ex_.close()


def run_profile_case(name: str):
    """A few launches of one kernel on a case sized for a profiler capture: larger than L2, well under
    a GB on the device.  Prints one JSON line with the CUDA-event time of the last launch."""
    from robogoat_b200 import ops
    import workloads
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
    elif name == "voxel_mean_runs":
        # the slab-ordered run path on a capture-sized case: 2^24 mixture points into 256^3 voxels of 0.2 m
        # (accumulators 335 MB > L2, 1.2 GB on the device in all)
        N = 1 << 24
        pts, feats = workloads.voxel_mixture_inputs(N, seed=0, device=dev)
        kw = dict(grid_min=[-25.6, -25.6, -25.6], voxel_size=0.2, grid_size=[256, 256, 256])
        fn = lambda: robocache.voxelize_pointcloud(pts, feats, mode="mean", **kw)
        units = {"N": N, "grid": "256^3"}
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
    elif name == "voxel_tsdf":
        # the benchmark's TSDF case: 4 x 65536 points on a sphere of radius 2 with outward normals into [4,128^3], 3-voxel truncation
        from robogoat_b200 import batched
        g = torch.Generator().manual_seed(5)
        sp = torch.randn(4, 65536, 3, generator=g)
        sp = sp / sp.norm(dim=2, keepdim=True)
        spd, nrm = (sp * 2.0).to(dev), sp.to(dev)
        fn = lambda: batched.voxelize_tsdf(spd, nrm, [128, 128, 128], 0.05, [-3.2, -3.2, -3.2], 0.15)
        units = {"B": 4, "N": 65536, "grid": "128^3"}
    elif name == "voxel_sparse":
        # the sparse reduction's send and merge kernels as one of 8 ranks would run them, with the owners' record lists
        # in this GPU's memory: a private 256^3 grid of 2^24 mixture points (335 MB of sums and counts), the occupied
        # voxels of the 7 other slabs appended to 7 lists, then 7 such lists merged into this rank's slab
        from robogoat_b200 import sharding
        N, Vv, R = 1 << 24, 256 ** 3, 8
        pts, feats = workloads.voxel_mixture_inputs(N, seed=0, device=dev)
        kw = dict(grid_min=[-25.6, -25.6, -25.6], voxel_size=0.2, grid_size=[256, 256, 256])
        g_, c_ = ops.voxelize_pointcloud_cuda(pts, feats, kw["grid_min"], kw["voxel_size"], kw["grid_size"], "mean", normalize=False)
        g_, c_ = g_.view(Vv, 4), c_.view(Vv)
        del pts, feats
        cap = Vv // R
        ids = torch.empty(R * cap, dtype=torch.int32, device=dev)
        sums = torch.empty(R * cap, 4, dtype=torch.float32, device=dev)
        cnts = torch.empty(R * cap, dtype=torch.int32, device=dev)
        nrec = torch.zeros(R, dtype=torch.int32, device=dev)
        cursors = torch.zeros(16, dtype=torch.int32, device=dev)
        overflow = torch.zeros(1, dtype=torch.int32, device=dev)
        others = list(range(1, R))

        def fn():
            ops.voxel_sparse_send_cuda(g_, c_, [sharding.slab_bounds(Vv, d, R) for d in others], cap,
                                       [ids.data_ptr() + d * cap * 4 for d in others], [sums.data_ptr() + d * cap * 16 for d in others],
                                       [cnts.data_ptr() + d * cap * 4 for d in others], [nrec.data_ptr() + d * 4 for d in others],
                                       cursors, overflow)
            # every list holds voxels of ITS slab; shift slab 1's list onto slab 0 would need new ids, so merge list d into
            # slab d of the private grid itself (same kernel, same access pattern as an owner's merge)
            for d in others[:1]:
                lo, hi = sharding.slab_bounds(Vv, d, R)
                ops.voxel_sparse_merge_cuda([ids.data_ptr() + d * cap * 4], [sums.data_ptr() + d * cap * 16], [cnts.data_ptr() + d * cap * 4],
                                            [nrec.data_ptr() + d * 4], cap, g_, c_, lo, hi, normalize=False)
        units = {"N": N, "grid": "256^3", "ranks_emulated": R}
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
                    help="run 4 launches of one kernel on a small case (resample, fusion, voxel_mean, voxel_count, voxel_occupancy, voxel_partition, voxel_partition_aligned, voxel_scatter_runs, voxel_mean_runs, voxel_sparse, voxel_tsdf; voxel_mean_full = headline size)")
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
