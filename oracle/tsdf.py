"""CPU restatement of the reference's truncated-signed-distance voxelisation - TEST INFRASTRUCTURE ONLY.

Parity status: UNPINNED.  The reference has no CPU path, test or golden vector for ``voxelize_tsdf``; this follows
its CUDA kernel (robocache/kernels/cutlass/point_cloud_voxelization.cu:278-376) line by line where that kernel's
result is well defined:

* voxel centre ``origin + (v + 0.5) * voxel_size``, offset ``centre - point``, ``dist = sqrt(dx*dx + dy*dy + dz*dz)``
  (lines 326-336), all in fp32, one rounding per operation, sums left to right;
* the voxel is touched when ``dist < truncation`` (line 338); its value is ``min(1, dist * (1/truncation))``,
  negative when ``dot(normal, centre - point) > 0`` (lines 340-356); its weight counts the touching points (line 373);
* per voxel the smallest magnitude wins (lines 362-371).

The kernel's compare-and-swap loop keeps the sign of whichever point wrote first, so with normals of both sides its
sign depends on thread order; here the sign is that of the closest point, and of the outside point on an exact tie.
Brute force over (point, voxel) pairs with numpy: for small cases only.
"""
from __future__ import annotations

from typing import Optional, Sequence, Tuple

import numpy as np


def voxelize_tsdf(points, normals: Optional[object], grid_size: Sequence[int], voxel_size: float, origin: Sequence[float],
                  truncation_distance: float) -> Tuple[np.ndarray, np.ndarray]:
    """points [B,N,3], normals [B,N,3] or None -> (tsdf [B,D,H,W] fp32, weights [B,D,H,W] fp32)."""
    pts = np.asarray(points, dtype=np.float32)
    nrm = None if normals is None else np.asarray(normals, dtype=np.float32)
    B, N, _ = pts.shape
    D, H, W = (int(v) for v in grid_size)
    f = np.float32
    vs, trunc = f(voxel_size), f(truncation_distance)
    inv_trunc = f(1.0) / trunc
    o = [f(v) for v in origin]
    cx = o[0] + (np.arange(W, dtype=np.float32) + f(0.5)) * vs           # [W]
    cy = o[1] + (np.arange(H, dtype=np.float32) + f(0.5)) * vs
    cz = o[2] + (np.arange(D, dtype=np.float32) + f(0.5)) * vs
    empty = np.uint32(0xFFFFFFFF)
    tsdf = np.zeros((B, D, H, W), dtype=np.float32)
    weights = np.zeros((B, D, H, W), dtype=np.float32)
    for b in range(B):
        keys = np.full((D, H, W), empty, dtype=np.uint32)
        wsum = np.zeros((D, H, W), dtype=np.float32)
        for i in range(N):
            x, y, z = pts[b, i]
            if not (np.isfinite(x) and np.isfinite(y) and np.isfinite(z)):
                continue
            dx = (cx - x)[None, None, :]
            dy = (cy - y)[None, :, None]
            dz = (cz - z)[:, None, None]
            with np.errstate(over="ignore"):                      # a far-away point squares to inf, as on the GPU
                dist = np.sqrt((dx * dx + dy * dy) + dz * dz)
            hit = dist < trunc
            if not hit.any():
                continue
            inside = np.zeros_like(hit)
            if nrm is not None:
                nx, ny, nz = nrm[b, i]
                inside = ((nx * dx + ny * dy) + nz * dz) > f(0.0)
            val = np.minimum(f(1.0), dist * inv_trunc).astype(np.float32)
            key = (val.view(np.uint32) << np.uint32(1)) | inside.astype(np.uint32)
            keys = np.where(hit, np.minimum(keys, key), keys)
            wsum = wsum + hit.astype(np.float32)
        mag = (keys >> np.uint32(1)).view(np.float32)
        out = np.where(keys & np.uint32(1), -mag, mag).astype(np.float32)
        tsdf[b] = np.where(keys == empty, f(0.0), out)
        weights[b] = wsum
    return tsdf, weights
