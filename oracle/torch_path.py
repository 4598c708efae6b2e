"""Torch restatement of the reference's CPU path, kept as the timed CPU baseline.  TEST INFRASTRUCTURE:
only tests and bench.py's CPU legs import it; no product path does.

The reference's CPU fallback is Python/torch (robocache/python/robocache/ops_fallback.py): a Python loop
over the batch with vectorised torch ops inside for resampling and fusion (:104-157, :59-101), and
floor / clamp / bincount / index_add_ for voxelisation (:160-258).  The reference checkout does not travel
to the GPU box, so its cost profile is restated here op for op - same torch calls in the same order, hence
the same rounding and the same speed - and checked bit for bit against fixtures the reference itself
produced (tests/golden, tests/test_oracle_golden.py).

The voxel function follows the fallback's own semantics (out-of-grid points are clamped to the border
voxels and the grid is indexed [x][y][z]); those differ from the reference's CUDA kernels, which is why it is
a timed baseline only and not the parity oracle.
"""
from __future__ import annotations

import torch


def interpolate_stream(features: torch.Tensor, source_times: torch.Tensor, target_times: torch.Tensor) -> torch.Tensor:
    """[B,S,D], [B,S], [B,T] -> [B,T,D]; ops_fallback.py:104-157 (one searchsorted per batch row)."""
    S = features.shape[1]
    rows = []
    for feat_b, st_b, tt_b in zip(features, source_times, target_times):
        hi = torch.searchsorted(st_b, tt_b).clamp(1, S - 1)
        lo = hi - 1
        t_lo, t_hi = st_b[lo], st_b[hi]
        w = ((tt_b - t_lo) / (t_hi - t_lo + 1e-8)).clamp(0, 1).unsqueeze(-1)
        rows.append(feat_b[lo] * (1 - w) + feat_b[hi] * w)
    return torch.stack(rows, dim=0)


def fuse_multimodal(s1, t1, s2, t2, s3, t3, target_times) -> torch.Tensor:
    """Three resampled streams side by side; ops_fallback.py:59-101."""
    return torch.cat([interpolate_stream(s1, t1, target_times), interpolate_stream(s2, t2, target_times),
                      interpolate_stream(s3, t3, target_times)], dim=-1)


def voxelize_pointcloud(points, features=None, grid_min=(-2.0, -2.0, -2.0), voxel_size=0.05,
                        grid_size=(128, 128, 128), mode="count") -> torch.Tensor:
    """ops_fallback.py:160-258: floor, clamp into the grid, x-major linear index, bincount / index_add_."""
    nx, ny, nz = (int(v) for v in grid_size)
    cell = torch.floor((points - torch.tensor([list(grid_min)], dtype=points.dtype)) / voxel_size).long()
    cell[:, 0].clamp_(0, nx - 1)
    cell[:, 1].clamp_(0, ny - 1)
    cell[:, 2].clamp_(0, nz - 1)
    lin = cell[:, 0] * ny * nz + cell[:, 1] * nz + cell[:, 2]
    V = nx * ny * nz
    if mode == "count":
        return torch.bincount(lin, minlength=V).reshape(nx, ny, nz).int()
    if mode == "occupancy":
        flat = torch.zeros(V, dtype=torch.int32)
        flat[lin] = 1
        return flat.reshape(nx, ny, nz)
    if features is None:
        raise ValueError("Features required for mean mode")
    F = features.shape[1]
    if mode == "mean":
        sums = torch.zeros(V, F, dtype=torch.float32).index_add_(0, lin, features.float())
        n = torch.bincount(lin, minlength=V).float() + 1e-8
        return (sums / n.unsqueeze(-1)).reshape(nx, ny, nz, F)
    if mode == "max":
        g = torch.full((V, F), float("-inf"), dtype=torch.float32)
        g.scatter_reduce_(0, lin.unsqueeze(-1).expand(-1, F), features.float(), reduce="amax", include_self=False)
        return torch.where(torch.isfinite(g), g, torch.zeros_like(g)).reshape(nx, ny, nz, F)
    raise ValueError(f"Unknown mode: {mode}")
