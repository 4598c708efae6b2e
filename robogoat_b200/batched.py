"""Batched voxel grids: ``[B, N, 3]`` clouds -> ``[B, D, H, W]`` float grids.

The older operator surface of the reference (robocache/kernels/cutlass/point_cloud_voxelization.h:59-92,
bound in point_cloud_voxelization_torch.cu:17-160) takes a batch of equally sized clouds and returns
float occupancy (0/1) or density (points per voxel) grids laid out ``[batch, depth(z), height(y),
width(x)]`` — the same z-major order the single-cloud operator uses.  Each item is binned by the
single-cloud kernel directly into its slice of one int32 batch grid; the result is converted once.
"""
from __future__ import annotations

import ctypes
from typing import Sequence

import torch

from . import _lib


def _voxelize_batched(points: torch.Tensor, grid_size: Sequence[int], voxel_size: float, origin: Sequence[float],
                      mode: int) -> torch.Tensor:
    if not points.is_cuda:
        raise RuntimeError("points must be on CUDA device")
    if points.dim() != 3 or points.shape[2] != 3:
        raise RuntimeError("points must have shape [batch, num_points, 3]")
    if len(grid_size) != 3:
        raise RuntimeError("grid_size must have 3 elements [depth, height, width]")
    if len(origin) != 3:
        raise RuntimeError("origin must have 3 elements [x, y, z]")
    if not voxel_size > 0:
        raise RuntimeError("voxel_size must be positive")
    depth, height, width = (int(v) for v in grid_size)
    B, N, _ = points.shape
    L = _lib.load()
    dev = points.device
    pts = points.to(torch.float32).contiguous()
    V = depth * height * width
    grid = torch.empty((B, depth, height, width), dtype=torch.int32, device=dev)
    gmin = (ctypes.c_float * 3)(*[float(v) for v in origin])
    gsz = (ctypes.c_int32 * 3)(width, height, depth)          # x, y, z extents
    stream = torch.cuda.current_stream(dev).cuda_stream
    for b in range(B):
        rc = L.rc_voxelize(pts.data_ptr() + b * N * 12, None, grid.data_ptr() + b * V * 4, None, N, 0, gmin,
                           float(voxel_size), gsz, mode, _lib.VOXEL_ZERO_INIT, dev.index, stream)
        _lib.check(rc, "voxelize (batched)")
    return grid.to(torch.float32)


def voxelize_occupancy_batched(points, grid_size, voxel_size, origin) -> torch.Tensor:
    """Float 0/1 occupancy, ``[B, D, H, W]`` (point_cloud_voxelization.h:59-70)."""
    return _voxelize_batched(points, _as_list(grid_size), float(voxel_size), _as_list(origin), _lib.VOXEL_OCCUPANCY)


def voxelize_density_batched(points, grid_size, voxel_size, origin) -> torch.Tensor:
    """Float points-per-voxel, ``[B, D, H, W]`` (point_cloud_voxelization.h:72-92)."""
    return _voxelize_batched(points, _as_list(grid_size), float(voxel_size), _as_list(origin), _lib.VOXEL_COUNT)


def _as_list(v):
    return v.tolist() if hasattr(v, "tolist") else list(v)
