"""ctypes binding of ``librobocache_b200.so`` (declared in ``include/robocache_b200.h``).

Loading is explicit and loud: a missing library raises, nothing falls back to a CPU or
torch implementation.
"""
from __future__ import annotations

import ctypes
import os
import threading

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "lib", "librobocache_b200.so")

RC_OK = 0
RC_DTYPE_F32 = 0
RC_DTYPE_BF16 = 1
RC_MAX_STREAMS = 8

VOXEL_COUNT = 0
VOXEL_OCCUPANCY = 1
VOXEL_MEAN = 2
VOXEL_MAX = 3
VOXEL_OCCUPANCY_U8 = 4

VOXEL_ZERO_INIT = 1
VOXEL_NO_NORMALIZE = 2
VOXEL_WARP_AGGREGATE = 4
VOXEL_SPARSE_OCCUPANCY = 8
STATIC_MAX_VOXELS = 1 << 21

BATCHED_OCCUPANCY = 0
BATCHED_DENSITY = 1
BATCHED_FEATURE_MEAN = 2
BATCHED_FEATURE_MAX = 3

OPT_BLOCK_KERNEL = 0
OPT_VOXEL_PASSES = 1
OPT_PART_ALIGNED_STORE = 2
OPT_BULK_WAIT_LIMIT = 3
OPT_GATHER_BULK_STAGE = 4
OPT_BUCKET_BULK_STORE = 5
OPT_SCATTER_OVERLAP = 6

# every symbol the header declares; the CPU test-suite checks the built library exports them all
EXPORTED_SYMBOLS = (
    "rc_resample", "rc_resample_strided", "rc_resample_ragged", "rc_fuse", "rc_fuse_strided", "rc_resample_brackets", "rc_voxelize", "rc_voxel_normalize", "rc_voxelize_mean_static",
    "rc_voxelize_ex", "rc_voxelize_scratch_bytes", "rc_voxel_partition", "rc_voxel_partition_count", "rc_voxel_partition_move", "rc_voxel_partition_scratch_bytes",
    "rc_voxel_scatter_ids", "rc_voxel_scatter_runs", "rc_peer_alloc", "rc_peer_open", "rc_peer_close", "rc_peer_free",
    "rc_voxelize_batched", "rc_point_cloud_bounds", "rc_voxelize_tsdf", "rc_voxel_bucket_block_records", "rc_voxel_bucket_exchange", "rc_voxel_scatter_buckets", "rc_voxel_sparse_send", "rc_voxel_sparse_merge", "rc_peer_barrier", "rc_set_option", "rc_bulk_wait_timeouts", "rc_strerror", "rc_last_cuda_error", "rc_abi_version",
)


class StreamDesc(ctypes.Structure):
    _fields_ = [("data", ctypes.c_void_p), ("times", ctypes.c_void_p),
                ("S", ctypes.c_int64), ("D", ctypes.c_int64)]


class LibraryNotBuilt(RuntimeError):
    pass


_lock = threading.Lock()
_lib = None


def _declare(L: ctypes.CDLL) -> None:
    vp, i64, i32, ci, f32, u32 = (ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32, ctypes.c_int,
                                  ctypes.c_float, ctypes.c_uint32)
    L.rc_resample.argtypes = [vp, vp, vp, vp, i64, i64, i64, i64, ci, ci, vp]
    L.rc_resample_strided.argtypes = [vp, vp, i64, vp, i64, vp, i64, i64, i64, i64, ci, ci, vp]
    L.rc_resample_strided.restype = ci
    L.rc_fuse_strided.argtypes = [ctypes.POINTER(StreamDesc), ctypes.POINTER(i64), ci, vp, i64, vp, i64, i64, ci, ci, vp]
    L.rc_fuse_strided.restype = ci
    L.rc_resample_ragged.argtypes = [vp, vp, vp, i64, vp, vp, i64, i64, i64, ci, ci, vp]
    L.rc_resample_ragged.restype = ci
    L.rc_fuse.argtypes = [ctypes.POINTER(StreamDesc), ci, vp, vp, i64, i64, ci, ci, vp]
    L.rc_resample_brackets.argtypes = [vp, vp, i64, i64, i64, vp, vp, vp, ci, vp]
    L.rc_voxelize.argtypes = [vp, vp, vp, vp, i64, i32, ctypes.POINTER(f32), f32,
                              ctypes.POINTER(i32), ci, u32, ci, vp]
    L.rc_voxel_normalize.argtypes = [vp, vp, i64, i64, i32, ci, vp]
    L.rc_voxelize_ex.argtypes = [vp, vp, vp, vp, i64, i32, ctypes.POINTER(f32), f32, ctypes.POINTER(i32), ci, u32, vp,
                                 ctypes.c_uint64, ci, vp]
    L.rc_voxelize_ex.restype = ci
    L.rc_voxelize_scratch_bytes.argtypes = [i64, i32, ctypes.POINTER(i32), ci]
    L.rc_voxelize_scratch_bytes.restype = ctypes.c_uint64
    L.rc_voxel_partition_scratch_bytes.argtypes = [i64, i32, ci]
    L.rc_voxel_partition_scratch_bytes.restype = ctypes.c_uint64
    fp, ip = ctypes.POINTER(f32), ctypes.POINTER(i32)
    L.rc_voxel_partition.argtypes = [vp, vp, i64, i32, fp, f32, ip, i32, i32, vp, vp, vp, vp, ctypes.c_uint64, ci, vp]
    L.rc_voxel_partition.restype = ci
    L.rc_voxel_partition_count.argtypes = [vp, i64, fp, f32, ip, i32, i32, vp, vp, ctypes.c_uint64, ci, vp]
    L.rc_voxel_partition_count.restype = ci
    L.rc_voxel_partition_move.argtypes = [vp, vp, i64, i32, fp, f32, ip, i32, i32, ctypes.POINTER(vp), ctypes.POINTER(vp),
                                          ctypes.POINTER(i64), vp, u32, vp, ctypes.c_uint64, ci, vp]
    L.rc_voxel_partition_move.restype = ci
    L.rc_voxel_scatter_runs.argtypes = [vp, vp, vp, vp, i32, i64, i64, ctypes.POINTER(i64), ctypes.POINTER(i64), ip, i32, i32,
                                        ci, u32, ci, vp]
    L.rc_voxel_scatter_runs.restype = ci
    L.rc_peer_alloc.argtypes = [ctypes.c_uint64, ci, ctypes.POINTER(vp), ctypes.c_char_p]
    L.rc_peer_open.argtypes = [ctypes.c_char_p, ci, ctypes.POINTER(vp)]
    L.rc_peer_close.argtypes = [vp, ci]
    L.rc_peer_free.argtypes = [vp, ci]
    for name in ("rc_peer_alloc", "rc_peer_open", "rc_peer_close", "rc_peer_free"):
        getattr(L, name).restype = ci
    L.rc_voxel_scatter_ids.argtypes = [vp, vp, vp, vp, i64, i32, i64, i64, ci, u32, ci, vp]
    L.rc_voxel_scatter_ids.restype = ci
    L.rc_voxelize_mean_static.argtypes = [vp, vp, vp, i64, i32, ctypes.POINTER(f32), f32, ctypes.POINTER(i32), ci, vp]
    L.rc_voxelize_batched.argtypes = [vp, vp, vp, vp, i64, i64, i32, ctypes.POINTER(f32), f32, ctypes.POINTER(i32), ci, u32, ci, vp]
    L.rc_voxelize_batched.restype = ci
    L.rc_point_cloud_bounds.argtypes = [vp, vp, vp, i64, i64, ci, vp]
    L.rc_point_cloud_bounds.restype = ci
    L.rc_voxelize_tsdf.argtypes = [vp, vp, vp, vp, i64, i64, ctypes.POINTER(f32), f32, ctypes.POINTER(i32), f32, ci, vp]
    L.rc_voxelize_tsdf.restype = ci
    L.rc_voxel_bucket_block_records.argtypes = [i32]
    L.rc_voxel_bucket_block_records.restype = i32
    L.rc_voxel_bucket_exchange.argtypes = [vp, vp, i64, ctypes.POINTER(f32), f32, ctypes.POINTER(i32), i32, i32, i64, i64, i64,
                                           ctypes.POINTER(vp), ctypes.POINTER(vp), ctypes.POINTER(vp), i32, ci, vp]
    L.rc_voxel_bucket_exchange.restype = ci
    L.rc_voxel_scatter_buckets.argtypes = [ctypes.POINTER(vp), ctypes.POINTER(vp), ctypes.POINTER(vp), i32, i64, i64, i32, vp, vp,
                                           i64, i64, u32, ci, vp]
    L.rc_voxel_scatter_buckets.restype = ci
    pvp = ctypes.POINTER(vp)
    L.rc_voxel_sparse_send.argtypes = [vp, vp, i32, ctypes.POINTER(i64), ctypes.POINTER(i64), i64, pvp, pvp, pvp, pvp, vp, vp, ci, vp]
    L.rc_voxel_sparse_send.restype = ci
    L.rc_voxel_sparse_merge.argtypes = [i32, pvp, pvp, pvp, pvp, i64, vp, vp, i64, i64, vp, u32, ci, vp]
    L.rc_voxel_sparse_merge.restype = ci
    L.rc_peer_barrier.argtypes = [pvp, i32, i32, u32, vp, i64, ci, vp]
    L.rc_peer_barrier.restype = ci
    for name in ("rc_resample", "rc_resample_strided", "rc_resample_ragged", "rc_fuse", "rc_fuse_strided", "rc_resample_brackets", "rc_voxelize", "rc_voxel_normalize", "rc_voxelize_mean_static",
                 "rc_last_cuda_error", "rc_abi_version"):
        getattr(L, name).restype = ci
    L.rc_set_option.argtypes = [ci, ci]
    L.rc_bulk_wait_timeouts.argtypes = [ci, ctypes.POINTER(u32)]
    L.rc_set_option.restype = ci
    L.rc_bulk_wait_timeouts.restype = ci
    L.rc_strerror.argtypes = [ci]
    L.rc_strerror.restype = ctypes.c_char_p


def load() -> ctypes.CDLL:
    """The CUDA library, loaded once.  Raises LibraryNotBuilt if it has not been compiled."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            if not os.path.exists(LIB_PATH):
                raise LibraryNotBuilt(
                    f"RoboCache CUDA kernels not available: {LIB_PATH} is missing. "
                    "Build it with `python -m robogoat_b200.build`; there is no CPU fallback.")
            L = ctypes.CDLL(LIB_PATH)
            _declare(L)
            _lib = L
    return _lib


def is_built() -> bool:
    return _lib is not None or os.path.exists(LIB_PATH)


def check(status: int, what: str) -> None:
    """Turn a non-zero rc_status into the exception the reference's bindings would raise."""
    if status == RC_OK:
        return
    L = load()
    msg = L.rc_strerror(status).decode()
    if status == 6:
        msg += f" (cudaError {L.rc_last_cuda_error()})"
    raise RuntimeError(f"{what}: {msg}")
