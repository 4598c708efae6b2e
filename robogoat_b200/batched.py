"""Batched voxel grids: ``[B, N, 3]`` clouds -> ``[B, D, H, W(, F)]`` float grids, and per-item bounds.

The older operator surface of the reference (robocache/kernels/cutlass/point_cloud_voxelization.h:59-157 and
:218-227, bound in point_cloud_voxelization_torch.cu:17-160) takes a batch of equally sized clouds and returns
float occupancy (0/1), density (points per voxel), feature-mean / feature-max or truncated-signed-distance grids laid out ``[batch, depth(z), height(y),
width(x)]`` — the same z-major order the single-cloud operator uses.  One kernel launch bins the whole batch
(the item index is folded into the voxel id) into one batch grid that was cleared with one fill.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence, Tuple

import torch

from . import _lib


def _as_list(v):
    return v.tolist() if hasattr(v, "tolist") else list(v)


def _check_cloud(points: torch.Tensor) -> None:
    if not points.is_cuda:
        raise RuntimeError("points must be on CUDA device")
    if points.dim() != 3 or points.shape[2] != 3:
        raise RuntimeError("points must have shape [batch, num_points, 3]")


def _voxelize_batched(points: torch.Tensor, features, grid_size: Sequence[int], voxel_size: float,
                      origin: Sequence[float], mode: int):
    _check_cloud(points)
    if len(grid_size) != 3:
        raise RuntimeError("grid_size must have 3 elements [depth, height, width]")
    if len(origin) != 3:
        raise RuntimeError("origin must have 3 elements [x, y, z]")
    if not voxel_size > 0:
        raise RuntimeError("voxel_size must be positive")
    depth, height, width = (int(v) for v in grid_size)
    B, N, _ = points.shape
    dev = points.device
    pts = points.to(torch.float32).contiguous()
    F, feats, counts = 0, None, None
    if mode in (_lib.BATCHED_FEATURE_MEAN, _lib.BATCHED_FEATURE_MAX):
        if features is None:
            raise RuntimeError("features required for mean/max modes")
        if not features.is_cuda or features.device != dev:
            raise RuntimeError("all tensors must be on the same CUDA device")
        if features.dim() != 3 or features.shape[0] != B or features.shape[1] != N:
            raise RuntimeError("features must have shape [batch, num_points, feature_dim]")
        F = features.shape[2]
        feats = features.to(torch.float32).contiguous()
        grid = torch.empty((B, depth, height, width, F), dtype=torch.float32, device=dev)
        if mode == _lib.BATCHED_FEATURE_MEAN:
            counts = torch.empty((B, depth, height, width), dtype=torch.int32, device=dev)
    else:
        grid = torch.empty((B, depth, height, width), dtype=torch.float32, device=dev)
    org = (ctypes.c_float * 3)(*[float(v) for v in origin])
    dhw = (ctypes.c_int32 * 3)(depth, height, width)
    rc = _lib.load().rc_voxelize_batched(pts.data_ptr(), feats.data_ptr() if feats is not None else None, grid.data_ptr(),
                                         counts.data_ptr() if counts is not None else None, B, N, F, org, float(voxel_size),
                                         dhw, mode, _lib.VOXEL_ZERO_INIT, dev.index,
                                         torch.cuda.current_stream(dev).cuda_stream)
    _lib.check(rc, "voxelize (batched)")
    return grid, counts


def voxelize_occupancy_batched(points, grid_size, voxel_size, origin) -> torch.Tensor:
    """Float 0/1 occupancy, ``[B, D, H, W]`` (point_cloud_voxelization.h:59-70)."""
    return _voxelize_batched(points, None, _as_list(grid_size), float(voxel_size), _as_list(origin), _lib.BATCHED_OCCUPANCY)[0]


def voxelize_density_batched(points, grid_size, voxel_size, origin) -> torch.Tensor:
    """Float points-per-voxel, ``[B, D, H, W]`` (point_cloud_voxelization.h:72-92)."""
    return _voxelize_batched(points, None, _as_list(grid_size), float(voxel_size), _as_list(origin), _lib.BATCHED_DENSITY)[0]


def voxelize_feature_mean_batched(points, features, grid_size, voxel_size, origin) -> torch.Tensor:
    """Per-voxel mean of the point features, ``[B, D, H, W, F]``, empty voxels 0 (point_cloud_voxelization.h:118-136)."""
    return _voxelize_batched(points, features, _as_list(grid_size), float(voxel_size), _as_list(origin),
                             _lib.BATCHED_FEATURE_MEAN)[0]


def voxelize_feature_max_batched(points, features, grid_size, voxel_size, origin) -> torch.Tensor:
    """Per-voxel maximum of the point features floored at 0, ``[B, D, H, W, F]``, empty voxels 0: what the reference's
    kernel computes by taking ``fmaxf`` against a zero-filled grid (point_cloud_voxelization.h:94-116, .cu:139-195).
    The single-cloud ``voxelize_pointcloud(..., mode="max")`` returns the true maximum instead."""
    return _voxelize_batched(points, features, _as_list(grid_size), float(voxel_size), _as_list(origin),
                             _lib.BATCHED_FEATURE_MAX)[0]


def compute_point_cloud_bounds(points: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(min_bounds, max_bounds)``, each ``[B, 3]``: the bounding box of every cloud of the batch
    (point_cloud_voxelization.h:218-227); an empty cloud yields (+1e10, -1e10) as the reference's kernel does."""
    _check_cloud(points)
    B, N, _ = points.shape
    dev = points.device
    pts = points.to(torch.float32).contiguous()
    lo = torch.empty((B, 3), dtype=torch.float32, device=dev)
    hi = torch.empty((B, 3), dtype=torch.float32, device=dev)
    rc = _lib.load().rc_point_cloud_bounds(pts.data_ptr(), lo.data_ptr(), hi.data_ptr(), B, N, dev.index,
                                           torch.cuda.current_stream(dev).cuda_stream)
    _lib.check(rc, "point_cloud_bounds")
    return lo, hi


def voxelize_tsdf(points: torch.Tensor, normals: Optional[torch.Tensor], grid_size, voxel_size: float, origin,
                  truncation_distance: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(tsdf, weights)``, each ``[B, D, H, W]`` fp32: for every voxel whose centre lies within ``truncation_distance``
    of a point, the smallest distance / truncation (negative where ``dot(normal, centre - point) > 0`` for the closest
    point, the reference kernel's sign rule) and the number of such points; 0 elsewhere
    (point_cloud_voxelization.h:146-173).  ``normals`` may be ``None`` (unsigned distances)."""
    _check_cloud(points)
    B, N, _ = points.shape
    dev = points.device
    pts = points.to(torch.float32).contiguous()
    nrm = None
    if normals is not None:
        if normals.shape != points.shape:
            raise ValueError(f"normals must have the points' shape {tuple(points.shape)}, got {tuple(normals.shape)}")
        if normals.device != dev:
            raise ValueError("normals must be on the points' device")
        nrm = normals.to(torch.float32).contiguous()
    depth, height, width = (int(v) for v in _as_list(grid_size))
    tsdf = torch.empty((B, depth, height, width), dtype=torch.float32, device=dev)
    weights = torch.empty((B, depth, height, width), dtype=torch.float32, device=dev)
    o = (ctypes.c_float * 3)(*[float(v) for v in _as_list(origin)])
    dhw = (ctypes.c_int32 * 3)(depth, height, width)
    rc = _lib.load().rc_voxelize_tsdf(pts.data_ptr(), nrm.data_ptr() if nrm is not None else None, tsdf.data_ptr(),
                                      weights.data_ptr(), B, N, o, float(voxel_size), dhw, float(truncation_distance),
                                      dev.index, torch.cuda.current_stream(dev).cuda_stream)
    _lib.check(rc, "voxelize_tsdf")
    return tsdf, weights
