"""CPU oracle for the RoboCache preprocessing hot path — TEST INFRASTRUCTURE ONLY.

ctypes bindings over ``oracle/robocache_oracle.c`` (a plain-C restatement of the
reference's CPU algorithms; every function there cites the reference lines it follows)
and, when it was built, over the reference's own C++ header compiled behind a C shim
(``oracle/_ref``).  Only the tests, the smoke check and the benchmark's CPU-baseline leg
import this package.  The shipped package never does: its operators raise when the CUDA
library is missing instead of falling back to anything here.

Parity status: pinned — see ``tests/test_oracle_golden.py`` (golden vectors produced by
the reference's ``ops_fallback`` module) and ``tests/test_oracle_ref_header.py`` (the
reference's ``cpu_reference.hpp`` voxel routines).

All functions take and return ``torch`` CPU tensors; bf16 data is passed through as-is.
"""
from __future__ import annotations

import ctypes
import os
import shutil
import subprocess
from typing import Optional, Sequence, Tuple

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "librobocache_oracle.so")
_REF_PATH = os.path.join(_HERE, "_ref", "librobocache_ref_cpu.so")

_REF_CUDA_PATH = os.path.join(_HERE, "_ref", "librobocache_ref_cuda.so")

_lib = None
_ref = None
_ref_cuda = None

_i64 = ctypes.c_int64
_i32 = ctypes.c_int32
_f32 = ctypes.c_float
_ptr = ctypes.c_void_p


def build(reference_root: Optional[str] = None) -> None:
    """Compile the oracle and, if a reference checkout is reachable, ``oracle/_ref``."""
    subprocess.run(["make", "-C", _HERE, "all"], check=True, capture_output=True)
    root = reference_root or os.environ.get("REFERENCE_ROOT") or os.path.abspath(os.path.join(_HERE, "..", "..", "reference"))
    if os.path.exists(os.path.join(root, "robocache", "validation", "cpu_reference.hpp")):
        subprocess.run(["make", "-C", _HERE, "ref", f"REFERENCE_ROOT={root}"],
                       check=True, capture_output=True)
    if os.path.exists(os.path.join(root, "robocache", "csrc", "cuda", "resample_kernel.cu")) and shutil.which("nvcc"):
        subprocess.run(["make", "-C", _HERE, "refcuda", f"REFERENCE_ROOT={root}"],
                       check=True, capture_output=True)


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        L = ctypes.CDLL(_LIB_PATH)
        L.orc_brackets.argtypes = [_ptr, _ptr, _i64, _i64, _i64, _ptr, _ptr, _ptr]
        L.orc_resample.argtypes = [_ptr, ctypes.c_int, _ptr, _ptr, _ptr, _i64, _i64, _i64, _i64,
                                   ctypes.c_int]
        L.orc_fuse3.argtypes = [_ptr, _ptr, _i64, _i64, _ptr, _ptr, _i64, _i64, _ptr, _ptr, _i64,
                                _i64, ctypes.c_int, _ptr, _ptr, _i64, _i64, ctypes.c_int]
        L.orc_voxel_ids.argtypes = [_ptr, _i64, _ptr, _f32, _ptr, _ptr]
        L.orc_voxelize_count.argtypes = [_ptr, _i64, _ptr, _f32, _ptr, ctypes.c_int, _ptr]
        L.orc_voxelize_mean.argtypes = [_ptr, _ptr, _i64, _i32, _ptr, _f32, _ptr, _ptr, _ptr, _ptr]
        L.orc_f32_to_bf16.argtypes = [_ptr, _ptr, _i64]
        L.orc_max_threads.restype = ctypes.c_int
        for f in ("orc_brackets", "orc_resample", "orc_fuse3", "orc_voxel_ids",
                  "orc_voxelize_count", "orc_voxelize_mean", "orc_f32_to_bf16"):
            getattr(L, f).restype = None
        _lib = L
    return _lib


def ref_lib() -> Optional[ctypes.CDLL]:
    """The reference's own C++ CPU header behind a C shim, or None if it was not built."""
    global _ref
    if _ref is None and os.path.exists(_REF_PATH):
        R = ctypes.CDLL(_REF_PATH)
        sig = [_ptr, _ptr, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
               _f32, _ptr]
        R.ref_voxelize_occupancy.argtypes = sig
        R.ref_voxelize_density.argtypes = sig
        R.ref_resample_f32.argtypes = [_ptr, _ptr, _ptr, _ptr] + [ctypes.c_int] * 4
        for f in ("ref_voxelize_occupancy", "ref_voxelize_density", "ref_resample_f32"):
            getattr(R, f).restype = None
        _ref = R
    return _ref


def ref_cuda_lib() -> Optional[ctypes.CDLL]:
    """The reference's own CUDA launchers compiled for sm_100a behind a C shim (comparator only), or None."""
    global _ref_cuda
    if _ref_cuda is None and os.path.exists(_REF_CUDA_PATH):
        R = ctypes.CDLL(_REF_CUDA_PATH)
        ci = ctypes.c_int
        R.launch_resample_bf16.argtypes = [_ptr, _ptr, _ptr, _ptr, ci, ci, ci, ci, _ptr]
        R.launch_resample_fp32.argtypes = [_ptr, _ptr, _ptr, _ptr, ci, ci, ci, ci, _ptr]
        R.refcuda_fuse.argtypes = [_ptr] * 8 + [ci] * 9 + [_ptr]
        R.refcuda_voxelize.argtypes = [_ptr, _ptr, _ptr, _ptr, ci, ci, _f32, _f32, _f32, _f32, ci, ci, ci, ci, _ptr]
        for f in ("launch_resample_bf16", "launch_resample_fp32", "refcuda_fuse", "refcuda_voxelize"):
            getattr(R, f).restype = None
        _ref_cuda = R
    return _ref_cuda


def max_threads() -> int:
    return int(lib().orc_max_threads())


# ----------------------------------------------------------------------------- helpers

def _f32c(t: torch.Tensor) -> torch.Tensor:
    return t.detach().to("cpu", torch.float32).contiguous()


def _data(t: torch.Tensor) -> Tuple[torch.Tensor, int]:
    """Feature tensor as the oracle reads it: bf16 stays bf16, everything else -> fp32."""
    t = t.detach().to("cpu")
    if t.dtype == torch.bfloat16:
        return t.contiguous(), 1
    return t.to(torch.float32).contiguous(), 0


def _p(t: torch.Tensor) -> int:
    return t.data_ptr()


def _farr(vals: Sequence[float]):
    return (ctypes.c_float * len(vals))(*[float(v) for v in vals])


def _iarr(vals: Sequence[int]):
    return (ctypes.c_int32 * len(vals))(*[int(v) for v in vals])


def round_to_bf16(x: torch.Tensor) -> torch.Tensor:
    """Round an fp32 tensor once to bf16, round-to-nearest-even (the C helper)."""
    x = _f32c(x)
    out = torch.empty(x.shape, dtype=torch.bfloat16)
    lib().orc_f32_to_bf16(_p(x), _p(out), x.numel())
    return out


# ----------------------------------------------------------------------------- resample

def brackets(source_times: torch.Tensor, target_times: torch.Tensor):
    """(left, right, weight) per target: int32 [B,T], int32 [B,T], fp32 [B,T]."""
    st, tt = _f32c(source_times), _f32c(target_times)
    B, S = st.shape
    T = tt.shape[1]
    left = torch.empty(B, T, dtype=torch.int32)
    right = torch.empty(B, T, dtype=torch.int32)
    w = torch.empty(B, T, dtype=torch.float32)
    lib().orc_brackets(_p(st), _p(tt), B, S, T, _p(left), _p(right), _p(w))
    return left, right, w


def resample_trajectories(source_data, source_times, target_times, threads: int = 1) -> torch.Tensor:
    """fp32 result of the reference's torch CPU path; [B,T,D]."""
    src, is_bf16 = _data(source_data)
    st, tt = _f32c(source_times), _f32c(target_times)
    B, S, D = src.shape
    T = tt.shape[1]
    out = torch.empty(B, T, D, dtype=torch.float32)
    lib().orc_resample(_p(src), is_bf16, _p(st), _p(tt), _p(out), B, S, T, D, threads)
    return out


def fuse_multimodal(s1, t1, s2, t2, s3, t3, target_times, threads: int = 1) -> torch.Tensor:
    """fp32 result of the reference's torch CPU fusion; [B,T,D1+D2+D3]."""
    d1, k1 = _data(s1)
    d2, k2 = _data(s2)
    d3, k3 = _data(s3)
    if not (k1 == k2 == k3):
        raise ValueError("Stream dtypes must match")
    t1, t2, t3, tt = _f32c(t1), _f32c(t2), _f32c(t3), _f32c(target_times)
    B, T = tt.shape
    out = torch.empty(B, T, d1.shape[2] + d2.shape[2] + d3.shape[2], dtype=torch.float32)
    lib().orc_fuse3(_p(d1), _p(t1), d1.shape[1], d1.shape[2],
                    _p(d2), _p(t2), d2.shape[1], d2.shape[2],
                    _p(d3), _p(t3), d3.shape[1], d3.shape[2],
                    k1, _p(tt), _p(out), B, T, threads)
    return out


# ----------------------------------------------------------------------------- voxels

def voxel_ids(points, grid_min, voxel_size, grid_size) -> torch.Tensor:
    """Linear z-major voxel id per point (int64), -1 for dropped points."""
    pts = _f32c(points)
    ids = torch.empty(pts.shape[0], dtype=torch.int64)
    lib().orc_voxel_ids(_p(pts), pts.shape[0], _farr(grid_min), float(voxel_size),
                        _iarr(grid_size), _p(ids))
    return ids


def voxelize_pointcloud(points, features=None, grid_min=(-10.0, -10.0, -10.0), voxel_size=0.1,
                        grid_size=(128, 128, 128), mode="occupancy", return_aux=False):
    """Voxel grid in the reference CUDA layout: a contiguous tensor shaped [gx,gy,gz]
    (or [gx,gy,gz,F]) whose flat index is vz*gx*gy + vy*gx + vx."""
    pts = _f32c(points)
    N = pts.shape[0]
    gx, gy, gz = [int(v) for v in grid_size]
    if mode in ("count", "occupancy"):
        grid = torch.empty(gx, gy, gz, dtype=torch.int32)
        lib().orc_voxelize_count(_p(pts), N, _farr(grid_min), float(voxel_size),
                                 _iarr(grid_size), 0 if mode == "count" else 1, _p(grid))
        return grid
    if mode == "mean":
        if features is None:
            raise ValueError("Features required for mean mode")
        feats = _f32c(features)
        F = feats.shape[1]
        grid = torch.empty(gx, gy, gz, F, dtype=torch.float32)
        counts = torch.empty(gx, gy, gz, dtype=torch.int32)
        sabs = torch.empty(gx, gy, gz, F, dtype=torch.float32)
        lib().orc_voxelize_mean(_p(pts), _p(feats), N, F, _farr(grid_min), float(voxel_size),
                                _iarr(grid_size), _p(grid), _p(counts), _p(sabs))
        return (grid, counts, sabs) if return_aux else grid
    raise ValueError(f"Unknown mode: {mode}")


def mean_tolerance(counts: torch.Tensor, sums_abs: torch.Tensor, expected: torch.Tensor) -> torch.Tensor:
    """Allowed |got - expected| per mean entry: 1e-5 relative plus an absolute floor of
    1e-6 times the mean magnitude of the summands (fp32 sums are order dependent)."""
    c = counts.clamp(min=1).to(torch.float32).unsqueeze(-1)
    return 1e-5 * expected.abs() + 1e-6 * (sums_abs / c)


# ----------------------------------------------------------------------------- reference header

def ref_header_voxelize(points, grid_min, voxel_size, grid_size, density: bool) -> Optional[torch.Tensor]:
    """The reference header's float occupancy / density grid (flat z-major), or None."""
    R = ref_lib()
    if R is None:
        return None
    pts = _f32c(points)
    gx, gy, gz = [int(v) for v in grid_size]
    grid = torch.empty(gx * gy * gz, dtype=torch.float32)
    fn = R.ref_voxelize_density if density else R.ref_voxelize_occupancy
    # header argument order: depth (z), height (y), width (x)
    fn(_p(pts), _p(grid), 1, pts.shape[0], gz, gy, gx, float(voxel_size), _farr(grid_min))
    return grid


# ----------------------------------------------------------------------------- reference CUDA kernels (comparator)

def ref_cuda_resample(source_data: torch.Tensor, source_times: torch.Tensor, target_times: torch.Tensor,
                      out: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """The reference's resample kernel (robocache/csrc/cuda/resample_kernel.cu) on CUDA tensors, or None."""
    R = ref_cuda_lib()
    if R is None:
        return None
    B, S, D = source_data.shape
    T = target_times.shape[1]
    if out is None:
        out = torch.empty((B, T, D), dtype=source_data.dtype, device=source_data.device)
    fn = R.launch_resample_bf16 if source_data.dtype == torch.bfloat16 else R.launch_resample_fp32
    fn(_p(source_data), _p(source_times), _p(target_times), _p(out), B, S, T, D,
       torch.cuda.current_stream(source_data.device).cuda_stream)
    return out


def ref_cuda_fuse(s1, t1, s2, t2, s3, t3, target_times, out: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """The reference's fusion kernel (robocache/csrc/cuda/multimodal_kernel.cu) on CUDA tensors, or None."""
    R = ref_cuda_lib()
    if R is None:
        return None
    B, T = target_times.shape
    if out is None:
        out = torch.empty((B, T, s1.shape[2] + s2.shape[2] + s3.shape[2]), dtype=s1.dtype, device=s1.device)
    R.refcuda_fuse(_p(s1), _p(t1), _p(s2), _p(t2), _p(s3), _p(t3), _p(target_times), _p(out), B, s1.shape[1], s1.shape[2],
                   s2.shape[1], s2.shape[2], s3.shape[1], s3.shape[2], T, 1 if s1.dtype == torch.bfloat16 else 0,
                   torch.cuda.current_stream(s1.device).cuda_stream)
    return out


def ref_cuda_voxelize(points, features, grid_min, voxel_size, grid_size, mode: str):
    """The reference's voxel kernels (robocache/csrc/cuda/voxelize_kernel.cu): returns (grid, counts or None), or None.
    Grids are zero-filled with torch first, as the reference binding does."""
    R = ref_cuda_lib()
    if R is None:
        return None
    code = {"count": 0, "occupancy": 1, "mean": 2}[mode]
    gx, gy, gz = [int(v) for v in grid_size]
    dev = points.device
    counts = None
    if mode == "mean":
        F = features.shape[1]
        grid = torch.zeros((gx, gy, gz, F), dtype=torch.float32, device=dev)
        counts = torch.zeros((gx, gy, gz), dtype=torch.int32, device=dev)
    else:
        F = 0
        grid = torch.zeros((gx, gy, gz), dtype=torch.int32, device=dev)
    R.refcuda_voxelize(_p(points), _p(features) if features is not None else None, _p(grid),
                       _p(counts) if counts is not None else None, points.shape[0], F, float(grid_min[0]),
                       float(grid_min[1]), float(grid_min[2]), float(voxel_size), gx, gy, gz, code,
                       torch.cuda.current_stream(dev).cuda_stream)
    return grid, counts
