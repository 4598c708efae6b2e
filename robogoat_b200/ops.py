"""Binding layer: validates torch tensors, allocates outputs and calls the C ABI.

These three functions mirror the reference's pybind11 entry points, with the same
checks and error texts:

* ``resample_trajectories_cuda``  — robocache/csrc/cpp/resample_ops.cpp:31-90
* ``fuse_multimodal_cuda``        — robocache/csrc/cpp/multimodal_ops.cpp:28-119
* ``voxelize_pointcloud_cuda``    — robocache/csrc/cpp/voxelize_ops.cpp:31-133

Outputs are allocated here with torch (device memory and streams are torch's job); the
kernels run on torch's current stream of the tensors' device.  There is no CPU path.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence, Tuple

import torch

from . import _lib

_MODES = {"count": _lib.VOXEL_COUNT, "occupancy": _lib.VOXEL_OCCUPANCY, "mean": _lib.VOXEL_MEAN,
          "max": _lib.VOXEL_MAX}


def _check(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream_ptr(device: torch.device) -> int:
    """cudaStream_t of torch's current stream on ``device`` (the raw accessor skips building a Stream object)."""
    if _raw_stream is not None:
        return _raw_stream(device.index)
    return torch.cuda.current_stream(device).cuda_stream


def _dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.bfloat16:
        return _lib.RC_DTYPE_BF16
    if dtype == torch.float32:
        return _lib.RC_DTYPE_F32
    raise RuntimeError("Unsupported dtype. Use float32 or bfloat16.")


def _times(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.float32).contiguous()


def _time_rows(t: torch.Tensor):
    """(tensor to keep alive, row stride in floats) of a [B, n] timestamp tensor.  fp32 rows with unit inner
    stride are used in place — in particular ``linspace(...).expand(B, -1)`` (row stride 0) is not copied."""
    if t.dtype == torch.float32 and (t.shape[1] <= 1 or t.stride(1) == 1):
        s0 = t.stride(0) if t.shape[0] > 1 else t.shape[1]
        if s0 == 0 or s0 >= t.shape[1]:
            return t, s0
    c = t.to(torch.float32).contiguous()
    return c, c.shape[1]


def resample_trajectories_cuda(source_data: torch.Tensor, source_times: torch.Tensor,
                               target_times: torch.Tensor) -> torch.Tensor:
    """[B,S,D] x [B,S] x [B,T] -> [B,T,D], dtype of ``source_data`` (fp32 or bf16)."""
    _check(source_data.is_cuda, "source_data must be CUDA tensor")
    _check(source_times.is_cuda, "source_times must be CUDA tensor")
    _check(target_times.is_cuda, "target_times must be CUDA tensor")
    _check(source_data.dim() == 3, "source_data must be 3D [B, S, D]")
    _check(source_times.dim() == 2, "source_times must be 2D [B, S]")
    _check(target_times.dim() == 2, "target_times must be 2D [B, T]")
    B, S, D = source_data.shape
    T = target_times.shape[1]
    _check(source_times.shape[0] == B, "Batch size mismatch")
    _check(source_times.shape[1] == S, "Source length mismatch")
    _check(target_times.shape[0] == B, "Batch size mismatch")
    _check(source_times.device == source_data.device and target_times.device == source_data.device,
           "all tensors must be on the same CUDA device")
    code = _dtype_code(source_data.dtype)
    _check(S >= 1 or T == 0 or B == 0, "source_data must have at least one timestep")

    L = _lib.load()
    src = source_data.contiguous()
    st, st_stride = _time_rows(source_times)
    tt, tt_stride = _time_rows(target_times)
    out = torch.empty((B, T, D), dtype=source_data.dtype, device=source_data.device)
    dev = source_data.device
    rc = L.rc_resample_strided(src.data_ptr(), st.data_ptr(), st_stride, tt.data_ptr(), tt_stride, out.data_ptr(),
                               B, S, T, D, code, dev.index, _stream_ptr(dev))
    _lib.check(rc, "resample_trajectories")
    return out


def fuse_streams_cuda(datas: Sequence[torch.Tensor], times: Sequence[torch.Tensor],
                      target_times: torch.Tensor) -> torch.Tensor:
    """N timestamped streams -> [B,T,sum(D_k)] in one launch (N <= 8)."""
    n = len(datas)
    if not (1 <= n <= _lib.RC_MAX_STREAMS and len(times) == n):
        raise RuntimeError(f"between 1 and {_lib.RC_MAX_STREAMS} streams are supported")
    # the checks of the reference binding, in its order; messages are only built on failure
    for k, d in enumerate(datas, 1):
        if not d.is_cuda:
            raise RuntimeError(f"stream{k}_data must be on CUDA device")
    for k, d in enumerate(datas, 1):
        if d.dim() != 3:
            raise RuntimeError(f"stream{k}_data must be 3D [B, S{k}, D{k}]")
    for k, t in enumerate(times, 1):
        if t.dim() != 2:
            raise RuntimeError(f"stream{k}_times must be 2D [B, S{k}]")
    if target_times.dim() != 2:
        raise RuntimeError("target_times must be 2D [B, T]")
    B = datas[0].shape[0]
    dtype0 = datas[0].dtype
    dev = datas[0].device
    T = target_times.shape[1]
    for d in datas:
        if d.shape[0] != B:
            raise RuntimeError("Batch size mismatch")
    for k, (d, t) in enumerate(zip(datas, times), 1):
        if t.shape[1] != d.shape[1]:
            raise RuntimeError(f"stream{k}_times length mismatch")
        if t.shape[0] != B:
            raise RuntimeError("Batch size mismatch")
    if target_times.shape[0] != B:
        raise RuntimeError("Batch size mismatch")
    for d in datas:
        if d.dtype != dtype0:
            raise RuntimeError("Stream dtypes must match")
    for x in (*datas, *times, target_times):
        if x.device != dev:
            raise RuntimeError("all tensors must be on the same CUDA device")
    code = _dtype_code(dtype0)
    for d in datas:
        if d.shape[1] < 1 and T != 0 and B != 0:
            raise RuntimeError("every stream must have at least one timestep")

    L = _lib.load()
    datas_c = [d.contiguous() for d in datas]
    times_c = [_time_rows(t) for t in times]
    tt, tt_stride = _time_rows(target_times)
    out = torch.empty((B, T, sum(d.shape[2] for d in datas)), dtype=datas[0].dtype, device=dev)
    descs = (_lib.StreamDesc * n)()
    strides = (ctypes.c_int64 * n)()
    for k in range(n):
        descs[k].data = datas_c[k].data_ptr()
        descs[k].times = times_c[k][0].data_ptr()
        descs[k].S = datas_c[k].shape[1]
        descs[k].D = datas_c[k].shape[2]
        strides[k] = times_c[k][1]
    rc = L.rc_fuse_strided(descs, strides, n, tt.data_ptr(), tt_stride, out.data_ptr(), B, T, code, dev.index,
                           _stream_ptr(dev))
    _lib.check(rc, "fuse_multimodal")
    return out


def fuse_multimodal_cuda(stream1_data, stream1_times, stream2_data, stream2_times, stream3_data,
                         stream3_times, target_times) -> torch.Tensor:
    """Three streams -> [B,T,D1+D2+D3]; slices in stream order."""
    return fuse_streams_cuda([stream1_data, stream2_data, stream3_data],
                             [stream1_times, stream2_times, stream3_times], target_times)


def resample_brackets_cuda(source_times: torch.Tensor, target_times: torch.Tensor):
    """(left int32, right int32, weight fp32), each [B,T]: the rows and weight the resampler uses."""
    _check(source_times.is_cuda and target_times.is_cuda, "times must be CUDA tensors")
    _check(source_times.dim() == 2 and target_times.dim() == 2, "times must be 2D")
    _check(source_times.shape[0] == target_times.shape[0], "Batch size mismatch")
    L = _lib.load()
    st, tt = _times(source_times), _times(target_times)
    B, S = st.shape
    T = tt.shape[1]
    dev = st.device
    left = torch.empty((B, T), dtype=torch.int32, device=dev)
    right = torch.empty((B, T), dtype=torch.int32, device=dev)
    w = torch.empty((B, T), dtype=torch.float32, device=dev)
    rc = L.rc_resample_brackets(st.data_ptr(), tt.data_ptr(), B, S, T, left.data_ptr(), right.data_ptr(),
                                w.data_ptr(), dev.index, _stream_ptr(dev))
    _lib.check(rc, "resample_brackets")
    return left, right, w


def voxelize_pointcloud_cuda(points: torch.Tensor, features: Optional[torch.Tensor], grid_min: Sequence[float],
                             voxel_size: float, grid_size: Sequence[int], mode: str, *,
                             normalize: bool = True, warp_aggregate: bool = False,
                             occupancy_dtype: torch.dtype = torch.int32) -> List[torch.Tensor]:
    """[N,3] points (+ [N,F] features) -> [grid] or, for mean mode, [grid, counts].

    The grid is a contiguous tensor shaped [gx,gy,gz] (or [gx,gy,gz,F]) whose flat index is
    vz*gx*gy + vy*gx + vx, as the reference's CUDA kernels lay it out.  ``normalize=False``
    leaves feature sums in the grid (partial grids of the multi-GPU harness);
    ``occupancy_dtype=torch.uint8`` selects the compact occupancy plane.
    """
    _check(points.is_cuda, "points must be on CUDA device")
    _check(points.dim() == 2, "points must be 2D [N, 3]")
    _check(points.shape[1] == 3, "points must have 3 coordinates (x, y, z)")
    _check(len(grid_min) == 3, "grid_min must have 3 elements [x, y, z]")
    _check(len(grid_size) == 3, "grid_size must have 3 elements [X, Y, Z]")
    _check(voxel_size > 0, "voxel_size must be positive")
    if mode not in _MODES:
        raise RuntimeError(f"Invalid mode: {mode}. Must be 'count', 'occupancy', 'mean', or 'max'")
    code = _MODES[mode]
    N = points.shape[0]
    gx, gy, gz = (int(v) for v in grid_size)
    _check(gx >= 0 and gy >= 0 and gz >= 0, "grid_size must be non-negative")
    dev = points.device
    F = 0
    feats = None
    if mode in ("mean", "max"):
        # the reference's API layer passes torch.empty(0) when the caller gave no features
        _check(features is not None and not (features.dim() == 1 and features.numel() == 0),
               "features required for mean/max modes")
        _check(features.is_cuda, "features must be on CUDA device")
        _check(features.dim() == 2, "features must be 2D [N, F]")
        _check(features.shape[0] == N, "features must match points length")
        _check(features.device == dev, "all tensors must be on the same CUDA device")
        F = features.shape[1]
        feats = features.to(torch.float32).contiguous()
    pts = points.to(torch.float32).contiguous()

    L = _lib.load()
    counts = None
    if mode in ("count", "occupancy"):
        if mode == "occupancy" and occupancy_dtype == torch.uint8:
            code = _lib.VOXEL_OCCUPANCY_U8
            grid = torch.empty((gx, gy, gz), dtype=torch.uint8, device=dev)
        else:
            grid = torch.empty((gx, gy, gz), dtype=torch.int32, device=dev)
    else:
        grid = torch.empty((gx, gy, gz, F), dtype=torch.float32, device=dev)
        if mode == "mean":
            counts = torch.empty((gx, gy, gz), dtype=torch.int32, device=dev)
    flags = _lib.VOXEL_ZERO_INIT
    if not normalize:
        flags |= _lib.VOXEL_NO_NORMALIZE
    if warp_aggregate:
        flags |= _lib.VOXEL_WARP_AGGREGATE
    gmin = (ctypes.c_float * 3)(*[float(v) for v in grid_min])
    gsz = (ctypes.c_int32 * 3)(gx, gy, gz)
    # large sparse grids in mean mode run a two-phase scatter that wants 4 bytes of scratch per point
    need = int(L.rc_voxelize_scratch_bytes(N, F, gsz, code))
    scratch = torch.empty(need, dtype=torch.uint8, device=dev) if need > 0 else None
    rc = L.rc_voxelize_ex(pts.data_ptr(), feats.data_ptr() if feats is not None else None, grid.data_ptr(),
                          counts.data_ptr() if counts is not None else None, N, F, gmin, float(voxel_size), gsz,
                          code, flags, scratch.data_ptr() if scratch is not None else None, need, dev.index,
                          _stream_ptr(dev))
    _lib.check(rc, "voxelize_pointcloud")
    return [grid, counts] if mode == "mean" else [grid]


def voxel_normalize_cuda(grid: torch.Tensor, counts: torch.Tensor, voxel_begin: int = 0,
                         voxel_end: Optional[int] = None) -> None:
    """In place: grid[v,:] *= 1/counts[v] for occupied voxels v in [voxel_begin, voxel_end)."""
    _check(grid.is_cuda and counts.is_cuda, "grid and counts must be on CUDA device")
    _check(grid.dtype == torch.float32 and counts.dtype == torch.int32, "grid must be float32, counts int32")
    _check(grid.is_contiguous() and counts.is_contiguous(), "grid and counts must be contiguous")
    V = counts.numel()
    F = grid.numel() // V if V else 0
    _check(V * F == grid.numel(), "grid must be [..., F] over the voxels of counts")
    end = V if voxel_end is None else int(voxel_end)
    dev = grid.device
    rc = _lib.load().rc_voxel_normalize(grid.data_ptr(), counts.data_ptr(), int(voxel_begin), end, F, dev.index,
                                        _stream_ptr(dev))
    _lib.check(rc, "voxel_normalize")


def _partition_inputs(points, features):
    _check(points.is_cuda and points.dim() == 2 and points.shape[1] == 3, "points must be a CUDA tensor [N, 3]")
    dev = points.device
    N = points.shape[0]
    pts = points.to(torch.float32).contiguous()
    feats = None
    if features is not None:
        _check(features.is_cuda and features.dim() == 2 and features.shape[0] == N, "features must be a CUDA tensor [N, F]")
        _check(features.device == dev, "all tensors must be on the same CUDA device")
        feats = features.to(torch.float32).contiguous()
    return pts, feats


def _check_parts(n_groups: int, parts_per_group: int) -> int:
    _check(n_groups >= 1 and parts_per_group >= 1 and n_groups * parts_per_group <= 64,
           "n_groups * parts_per_group must be in [1, 64]")
    return n_groups * parts_per_group


def voxel_partition_cuda(points: torch.Tensor, features: Optional[torch.Tensor], grid_min: Sequence[float],
                         voxel_size: float, grid_size: Sequence[int], n_groups: int, parts_per_group: int = 1):
    """Stable partition of a cloud's in-grid points by the part that owns their voxel.

    The voxel ids are cut into ``n_groups`` contiguous ranges of ceil(V / n_groups), each into
    ``parts_per_group`` sub-ranges; part = group * parts_per_group + sub.  Returns
    ``(ids [N] int32, features [N,F] or None, part_counts [parts] int64)``, all on the device: the first
    ``part_counts.sum()`` entries hold part 0's points, then part 1's, ... in input order; the rest is
    unwritten.  Reading ``part_counts`` on the host is the caller's synchronisation point.
    """
    P = _check_parts(int(n_groups), int(parts_per_group))
    pts, feats = _partition_inputs(points, features)
    dev, N = pts.device, pts.shape[0]
    F = feats.shape[1] if feats is not None else 0
    L = _lib.load()
    ids = torch.empty(N, dtype=torch.int32, device=dev)
    feats_out = torch.empty((N, F), dtype=torch.float32, device=dev) if feats is not None else None
    part_counts = torch.empty(P, dtype=torch.int64, device=dev)
    need = int(L.rc_voxel_partition_scratch_bytes(N, P, dev.index))
    scratch = torch.empty(max(need, 16), dtype=torch.uint8, device=dev)
    gmin = (ctypes.c_float * 3)(*[float(v) for v in grid_min])
    gsz = (ctypes.c_int32 * 3)(*[int(v) for v in grid_size])
    rc = L.rc_voxel_partition(pts.data_ptr(), feats.data_ptr() if feats is not None else None, N, F, gmin,
                              float(voxel_size), gsz, int(n_groups), int(parts_per_group), ids.data_ptr(),
                              feats_out.data_ptr() if feats_out is not None else None, part_counts.data_ptr(),
                              scratch.data_ptr(), need, dev.index, _stream_ptr(dev))
    _lib.check(rc, "voxel_partition")
    return ids, feats_out, part_counts


def voxel_partition_count_cuda(points: torch.Tensor, grid_min: Sequence[float], voxel_size: float,
                               grid_size: Sequence[int], n_groups: int, parts_per_group: int = 1):
    """First half of the partition: ``(part_counts [parts] int64 on the device, scratch)``.  Hand ``scratch``
    unchanged to ``voxel_partition_move_cuda`` for the same points."""
    P = _check_parts(int(n_groups), int(parts_per_group))
    pts, _ = _partition_inputs(points, None)
    dev, N = pts.device, pts.shape[0]
    L = _lib.load()
    part_counts = torch.empty(P, dtype=torch.int64, device=dev)
    need = int(L.rc_voxel_partition_scratch_bytes(N, P, dev.index))
    scratch = torch.empty(max(need, 16), dtype=torch.uint8, device=dev)
    gmin = (ctypes.c_float * 3)(*[float(v) for v in grid_min])
    gsz = (ctypes.c_int32 * 3)(*[int(v) for v in grid_size])
    rc = L.rc_voxel_partition_count(pts.data_ptr(), N, gmin, float(voxel_size), gsz, int(n_groups), int(parts_per_group),
                                    part_counts.data_ptr(), scratch.data_ptr(), need, dev.index, _stream_ptr(dev))
    _lib.check(rc, "voxel_partition_count")
    return part_counts, scratch


def voxel_partition_move_cuda(points: torch.Tensor, features: Optional[torch.Tensor], grid_min: Sequence[float],
                              voxel_size: float, grid_size: Sequence[int], n_groups: int, parts_per_group: int,
                              dest_ids: Sequence[int], dest_features: Optional[Sequence[int]], dest_start: Sequence[int],
                              scratch: torch.Tensor, remote: bool = False) -> None:
    """Second half: writes part p's voxel ids to the device address ``dest_ids[p]`` (and feature rows to
    ``dest_features[p]``) from slot ``dest_start[p]`` on.  The addresses may belong to peer GPUs' buffers
    (``PeerBuffer``) - say so with ``remote=True`` and every warp store is shaped as one aligned 128-byte group, which is
    what stores over NVLink need; the caller guarantees room for the counted points."""
    P = _check_parts(int(n_groups), int(parts_per_group))
    _check(len(dest_ids) == P and len(dest_start) == P, "one destination and start slot per part")
    pts, feats = _partition_inputs(points, features if dest_features is not None else None)
    dev, N = pts.device, pts.shape[0]
    F = feats.shape[1] if feats is not None else 0
    L = _lib.load()
    VP = ctypes.c_void_p * P
    ids_arr = VP(*[int(a) for a in dest_ids])
    feats_arr = VP(*[int(a) for a in dest_features]) if feats is not None else None
    start_arr = (ctypes.c_int64 * P)(*[int(v) for v in dest_start])
    gmin = (ctypes.c_float * 3)(*[float(v) for v in grid_min])
    gsz = (ctypes.c_int32 * 3)(*[int(v) for v in grid_size])
    rc = L.rc_voxel_partition_move(pts.data_ptr(), feats.data_ptr() if feats is not None else None, N, F, gmin,
                                   float(voxel_size), gsz, int(n_groups), int(parts_per_group), ids_arr, feats_arr,
                                   start_arr, None, 1 if remote else 0, scratch.data_ptr(), scratch.numel(), dev.index,
                                   _stream_ptr(dev))
    _lib.check(rc, "voxel_partition_move")


def voxel_bucket_exchange_cuda(points: torch.Tensor, features: torch.Tensor, grid_min: Sequence[float], voxel_size: float,
                               grid_size: Sequence[int], n_groups: int, parts_per_group: int, chunks: int, first_block: int,
                               pool_blocks: int, dest_ids: Sequence[int], dest_features: Sequence[int],
                               dest_runs: Sequence[int], ctas_per_sm: int = 0) -> None:
    """Bucket a cloud by (owner, sub-range of the owner's slab): owner d's records of chunk c go to block
    ``first_block + c`` of pool d (device addresses, possibly of peer GPUs' buffers), with the run table beside them.
    Mean mode, four feature channels; see ``rc_voxel_bucket_exchange`` in the header for the layout."""
    _check(int(n_groups) * int(parts_per_group) <= 16, "n_groups * parts_per_group must be at most 16")
    pts, feats = _partition_inputs(points, features)
    _check(feats is not None and feats.shape[1] == 4, "the bucket exchange takes four feature channels")
    _check(len(dest_ids) == n_groups and len(dest_features) == n_groups and len(dest_runs) == n_groups,
           "one pool and one run table per owner")
    dev = pts.device
    VP = ctypes.c_void_p * int(n_groups)
    gmin = (ctypes.c_float * 3)(*[float(v) for v in grid_min])
    gsz = (ctypes.c_int32 * 3)(*[int(v) for v in grid_size])
    rc = _lib.load().rc_voxel_bucket_exchange(pts.data_ptr(), feats.data_ptr(), pts.shape[0], gmin, float(voxel_size), gsz,
                                              int(n_groups), int(parts_per_group), int(chunks), int(first_block),
                                              int(pool_blocks), VP(*[int(a) for a in dest_ids]),
                                              VP(*[int(a) for a in dest_features]), VP(*[int(a) for a in dest_runs]),
                                              int(ctas_per_sm), dev.index, _stream_ptr(dev))
    _lib.check(rc, "voxel_bucket_exchange")


def voxel_scatter_buckets_cuda(pool_ids: Sequence[int], pool_features: Sequence[int], runs: Sequence[int],
                               blocks_per_source: int, parts_per_group: int, device: torch.device, id_begin: int,
                               id_end: int, *, normalize: bool = True, table_row_blocks: int = 0, zero_init: bool = True,
                               out: Optional[List[torch.Tensor]] = None) -> List[torch.Tensor]:
    """The owner's side of the bucket exchange: accumulate the pools of every source (device addresses of their ids,
    feature rows and run tables; they may lie in other GPUs' memory) into the slab [id_begin, id_end); returns
    ``[grid fp32 [voxels, 4], counts int32 [voxels]]``.  ``out``: accumulators from ``voxel_slab_buffers`` to add into
    (with ``zero_init=False`` they keep what earlier calls accumulated); ``table_row_blocks``: row length of the run
    tables when a source is a window of a larger pool; an empty source list only clears / normalises."""
    device = torch.device(device)
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    n = len(pool_ids)
    _check(len(pool_features) == n and len(runs) == n and 0 <= n <= 16, "one pool and one run table per source (at most 16)")
    nvox = int(id_end) - int(id_begin)
    _check(nvox >= 0 and id_begin >= 0, "bad voxel range")
    grid, counts = out if out is not None else voxel_slab_buffers(nvox, 4, "mean", device)
    _check(grid.shape == (nvox, 4) and counts.shape == (nvox,) and grid.dtype == torch.float32 and counts.dtype == torch.int32
           and grid.is_contiguous() and counts.is_contiguous() and grid.device == device and counts.device == device,
           "out must be the slab's [grid fp32 [voxels, 4], counts int32 [voxels]] on the device")
    flags = (_lib.VOXEL_ZERO_INIT if zero_init else 0) | (0 if normalize else _lib.VOXEL_NO_NORMALIZE)
    VP = ctypes.c_void_p * max(n, 1)
    rc = _lib.load().rc_voxel_scatter_buckets(VP(*[int(a) for a in pool_ids]), VP(*[int(a) for a in pool_features]),
                                              VP(*[int(a) for a in runs]), n, int(blocks_per_source), int(table_row_blocks),
                                              int(parts_per_group),
                                              grid.data_ptr() if nvox else None, counts.data_ptr() if nvox else None,
                                              int(id_begin), int(id_end), flags, device.index, _stream_ptr(device))
    _lib.check(rc, "voxel_scatter_buckets")
    return [grid, counts]


def voxel_sparse_send_cuda(grid: Optional[torch.Tensor], counts: torch.Tensor, ranges: Sequence[Tuple[int, int]], capacity: int,
                           dest_ids: Sequence[int], dest_sums: Sequence[int], dest_counts: Sequence[int],
                           dest_nrec: Sequence[int], cursors: torch.Tensor, overflow: Optional[torch.Tensor]) -> None:
    """Append the occupied voxels of every range of a partial grid (``grid`` fp32 [V, 4] feature sums, ``counts`` int32
    [V]) to the record list of that range (device addresses, possibly peer memory) and publish the record numbers;
    see ``rc_voxel_sparse_send``.  ``cursors``: int32 [len(ranges)] scratch; ``overflow``: int32 [1] flag.  Count mode:
    ``grid=None`` and ``dest_sums`` all ``None`` - the records are (voxel id, count)."""
    n = len(ranges)
    _check(len(dest_ids) == n and len(dest_sums) == n and len(dest_counts) == n and len(dest_nrec) == n and n <= 16,
           "one record list per range (at most 16)")
    _check(counts.is_cuda and counts.dtype == torch.int32 and counts.is_contiguous(), "counts must be int32 [V] on a CUDA device")
    _check(grid is None or (grid.dtype == torch.float32 and grid.is_contiguous() and grid.numel() == counts.numel() * 4
                            and counts.device == grid.device), "grid must be fp32 [V, 4] sums on the counts' device")
    _check(cursors.dtype == torch.int32 and cursors.numel() >= n and cursors.device == counts.device, "cursors: int32 [ranges]")
    dev = counts.device
    VP = ctypes.c_void_p * max(n, 1)
    I64 = ctypes.c_int64 * max(n, 1)
    opt = lambda p: None if p is None else int(p)
    rc = _lib.load().rc_voxel_sparse_send(grid.data_ptr() if grid is not None else None, counts.data_ptr(), n,
                                          I64(*[int(a) for a, _ in ranges]),
                                          I64(*[int(b) for _, b in ranges]), int(capacity), VP(*[int(p) for p in dest_ids]),
                                          VP(*[opt(p) for p in dest_sums]), VP(*[int(p) for p in dest_counts]),
                                          VP(*[int(p) for p in dest_nrec]), cursors.data_ptr(),
                                          overflow.data_ptr() if overflow is not None else None, dev.index, _stream_ptr(dev))
    _lib.check(rc, "voxel_sparse_send")


def voxel_sparse_merge_cuda(src_ids: Sequence[int], src_sums: Sequence[int], src_counts: Sequence[int], src_nrec: Sequence[int],
                            capacity: int, grid: Optional[torch.Tensor], counts: torch.Tensor, id_begin: int, id_end: int, *,
                            normalize: bool = True, overflow: Optional[torch.Tensor] = None, occupancy: bool = False) -> None:
    """Add the record lists an owner received (device addresses) to its slab [id_begin, id_end) of its own partial grid
    (``grid`` fp32 [V, 4], ``counts`` int32 [V]: the FULL grid) and normalise the slab; see ``rc_voxel_sparse_merge``.
    Count mode: ``grid=None`` and ``src_sums`` all ``None``.  ``overflow``: int32 [1] flag that is set (never cleared)
    when a source reports more records than its list holds.  ``occupancy``: count mode storing 1 per received voxel."""
    n = len(src_ids)
    _check(len(src_sums) == n and len(src_counts) == n and len(src_nrec) == n and n <= 16, "one record list per source (at most 16)")
    _check(0 <= id_begin <= id_end <= counts.numel(), "bad voxel range")
    dev = counts.device
    VP = ctypes.c_void_p * max(n, 1)
    opt = lambda p: None if p is None else int(p)
    rc = _lib.load().rc_voxel_sparse_merge(n, VP(*[int(p) for p in src_ids]), VP(*[opt(p) for p in src_sums]),
                                           VP(*[int(p) for p in src_counts]), VP(*[int(p) for p in src_nrec]), int(capacity),
                                           grid.data_ptr() + int(id_begin) * 16 if grid is not None else None,
                                           counts.data_ptr() + int(id_begin) * 4,
                                           int(id_begin), int(id_end), overflow.data_ptr() if overflow is not None else None,
                                           (0 if normalize else _lib.VOXEL_NO_NORMALIZE) | (_lib.VOXEL_SPARSE_OCCUPANCY if occupancy else 0),
                                           dev.index, _stream_ptr(dev))
    _lib.check(rc, "voxel_sparse_merge")


def voxel_slab_buffers(n_voxels: int, feature_width: int, mode: str, device: torch.device) -> List[torch.Tensor]:
    """Uninitialised accumulators of a slab: ``[grid]`` (int32 [n]) or, for mean mode, ``[grid fp32 [n, F], counts int32 [n]]``."""
    if mode == "mean":
        return [torch.empty((n_voxels, feature_width), dtype=torch.float32, device=device),
                torch.empty(n_voxels, dtype=torch.int32, device=device)]
    return [torch.empty(n_voxels, dtype=torch.int32, device=device)]


def voxel_scatter_runs_cuda(ids_ptr: int, features_ptr: Optional[int], device: torch.device, feature_width: int,
                            id_begin: int, id_end: int, runs: Sequence[Tuple[int, int, int]], n_passes: int, mode: str,
                            *, normalize: bool = True, out: Optional[List[torch.Tensor]] = None) -> List[torch.Tensor]:
    """Accumulate records that arrive as runs into the slab of voxels [id_begin, id_end).

    ``ids_ptr`` / ``features_ptr`` are device addresses of the int32 id list and the fp32 [., F] feature rows
    (a torch tensor's ``data_ptr()`` or a ``PeerBuffer``); ``runs`` lists ``(first record, records, pass)``.
    The runs of pass 0 are accumulated first, then pass 1, ...  Returns ``[grid]`` or ``[grid, counts]`` as
    ``voxel_scatter_ids_cuda``.  ``out``: accumulators from ``voxel_slab_buffers`` that the caller has already
    cleared (e.g. on another stream while the records were still travelling); they are not cleared again.
    """
    if mode not in ("count", "occupancy", "mean"):
        raise RuntimeError(f"Invalid mode: {mode}. The run scatter supports 'count', 'occupancy' and 'mean'")
    device = torch.device(device)
    if device.index is None:                # "cuda" without an ordinal: the current device
        device = torch.device("cuda", torch.cuda.current_device())
    nvox = int(id_end) - int(id_begin)
    _check(nvox >= 0 and id_begin >= 0, "bad voxel range")
    F = int(feature_width) if mode == "mean" else 0
    if out is None:
        bufs = voxel_slab_buffers(nvox, F, mode, device)
    else:
        bufs = list(out)
        _check(bufs[0].is_contiguous() and bufs[0].numel() == (nvox * F if mode == "mean" else nvox), "out does not match the slab")
    grid = bufs[0]
    counts = bufs[1] if mode == "mean" else None
    n = len(runs)
    rb = (ctypes.c_int64 * max(n, 1))(*[int(r[0]) for r in runs])
    rcnt = (ctypes.c_int64 * max(n, 1))(*[int(r[1]) for r in runs])
    rp = (ctypes.c_int32 * max(n, 1))(*[int(r[2]) for r in runs])
    flags = (_lib.VOXEL_ZERO_INIT if out is None else 0) | (0 if normalize else _lib.VOXEL_NO_NORMALIZE)
    rc = _lib.load().rc_voxel_scatter_runs(ids_ptr or None, features_ptr or None, grid.data_ptr() if grid.numel() else None,
                                           counts.data_ptr() if counts is not None and nvox else None, F, int(id_begin),
                                           int(id_end), rb, rcnt, rp, n, int(n_passes), _MODES[mode], flags, device.index,
                                           _stream_ptr(device))
    _lib.check(rc, "voxel_scatter_runs")
    return [grid, counts] if mode == "mean" else [grid]


def voxel_scatter_ids_cuda(ids: torch.Tensor, features: Optional[torch.Tensor], id_begin: int, id_end: int,
                           mode: str, *, feature_width: int = 0, normalize: bool = True) -> List[torch.Tensor]:
    """Accumulate points given as (voxel id, feature row) into the slab of voxels [id_begin, id_end).

    Returns ``[grid]`` (int32 [id_end-id_begin] for count / occupancy) or ``[grid, counts]`` (fp32
    [id_end-id_begin, F] and int32 counts for mean).  Ids outside the range are ignored.
    """
    _check(ids.is_cuda and ids.dtype == torch.int32 and ids.dim() == 1 and ids.is_contiguous(),
           "ids must be a contiguous int32 CUDA vector")
    if mode not in ("count", "occupancy", "mean"):
        raise RuntimeError(f"Invalid mode: {mode}. The id scatter supports 'count', 'occupancy' and 'mean'")
    dev = ids.device
    M = ids.numel()
    nvox = int(id_end) - int(id_begin)
    _check(nvox >= 0 and id_begin >= 0, "bad voxel range")
    F = 0
    feats = None
    counts = None
    if mode == "mean":
        _check(features is not None or M == 0, "features required for mean mode")
        if features is not None:
            _check(features.is_cuda and features.dim() == 2 and features.shape[0] == M, "features must be [M, F] on CUDA")
            feats = features.to(torch.float32).contiguous()
            F = feats.shape[1]
        else:
            F = int(feature_width)
        grid = torch.empty((nvox, F), dtype=torch.float32, device=dev)
        counts = torch.empty(nvox, dtype=torch.int32, device=dev)
    else:
        grid = torch.empty(nvox, dtype=torch.int32, device=dev)
    flags = _lib.VOXEL_ZERO_INIT | (0 if normalize else _lib.VOXEL_NO_NORMALIZE)
    rc = _lib.load().rc_voxel_scatter_ids(ids.data_ptr() if M else None, feats.data_ptr() if feats is not None else None,
                                          grid.data_ptr() if grid.numel() else None,
                                          counts.data_ptr() if counts is not None and nvox else None, M, F,
                                          int(id_begin), int(id_end), _MODES[mode], flags, dev.index, _stream_ptr(dev))
    _lib.check(rc, "voxel_scatter_ids")
    return [grid, counts] if mode == "mean" else [grid]


def resample_ragged_cuda(source_rows: torch.Tensor, source_times: torch.Tensor, row_offsets: torch.Tensor,
                         target_times: torch.Tensor, max_len: Optional[int] = None) -> torch.Tensor:
    """Resample variable-length items that are packed back to back, without padding them.

    source_rows [sum S_b, D] (bf16/fp32), source_times [sum S_b], row_offsets [B+1] (int64, ascending,
    row_offsets[0] = 0), target_times [B, T] -> [B, T, D].  Equal to padding every item with its last step
    (as robocache/python/robocache/datasets/rtx_loader.py:214-221 does) and resampling the padded batch.
    ``max_len``: an upper bound of the item lengths; computed from the offsets (one host sync) when omitted.
    """
    _check(source_rows.is_cuda and source_times.is_cuda and row_offsets.is_cuda and target_times.is_cuda,
           "all tensors must be CUDA tensors")
    _check(source_rows.dim() == 2, "source_rows must be 2D [sum S, D]")
    _check(source_times.dim() == 1 and source_times.shape[0] == source_rows.shape[0],
           "source_times must be 1D with one entry per source row")
    _check(target_times.dim() == 2, "target_times must be 2D [B, T]")
    B, T = target_times.shape
    _check(row_offsets.dim() == 1 and row_offsets.shape[0] == B + 1, "row_offsets must have B+1 entries")
    code = _dtype_code(source_rows.dtype)
    dev = source_rows.device
    offs = row_offsets.to(torch.int64).contiguous()
    if max_len is None:
        max_len = int((offs[1:] - offs[:-1]).max().item()) if B > 0 else 0
    D = source_rows.shape[1]
    L = _lib.load()
    src = source_rows.contiguous()
    st, tt = _times(source_times), _times(target_times)
    out = torch.empty((B, T, D), dtype=source_rows.dtype, device=dev)
    rc = L.rc_resample_ragged(src.data_ptr(), st.data_ptr(), offs.data_ptr(), int(max_len), tt.data_ptr(), out.data_ptr(),
                              B, T, D, code, dev.index, _stream_ptr(dev))
    _lib.check(rc, "resample_ragged")
    return out
