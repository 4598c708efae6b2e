"""Seeded synthetic inputs with the shapes and value distributions of the headline configurations,
plus the byte accounting used for throughput figures.

Everything is generated with an explicit ``torch.Generator`` so that the CUDA path, the CPU oracle
and the benchmark see identical tensors.  Large cases can be generated directly on the GPU
(``device='cuda'``); parity tests generate on the CPU and copy.
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch


def _gen(seed: int, device) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return g


def cumsum_times(B: int, S: int, g: torch.Generator, device="cpu") -> torch.Tensor:
    """Per-row source timestamps: cumsum of U(0.5,1.5) increments, normalised to [0,1]."""
    inc = torch.rand(B, S, generator=g, device=device) + 0.5
    st = inc.cumsum(1)
    if S == 1:
        return torch.zeros(B, 1, device=device)
    return ((st - st[:, :1]) / (st[:, -1:] - st[:, :1])).contiguous()


def resample_inputs(B=32, S=500, D=256, T=250, dtype=torch.float32, irregular_targets=False, seed=0,
                    device="cpu") -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Trajectory resampling inputs.  ``irregular_targets=False``: linspace(0,1,T) shared by the
    batch (the fp32 CPU-sized case); ``True``: sorted U(0,1) draws per row (the bf16 B=4096 case)."""
    g = _gen(seed, device)
    st = cumsum_times(B, S, g, device)
    src = torch.randn(B, S, D, generator=g, device=device, dtype=torch.float32).to(dtype)
    if irregular_targets:
        tt = torch.sort(torch.rand(B, T, generator=g, device=device), dim=1).values.contiguous()
    else:
        tt = torch.linspace(0, 1, T, device=device).expand(B, -1).contiguous()
    return src, st, tt


FUSION_STREAMS = ((30, 512), (100, 64), (200, 12))  # (length, width) of vision, proprioception, IMU


def fusion_inputs(B=4, T=50, dtype=torch.bfloat16, seed=0, device="cpu", streams=FUSION_STREAMS):
    """Three streams timestamped linspace(0,1,n) + N(0,1e-3) jitter, sorted; targets linspace(0,1,T)."""
    g = _gen(seed, device)
    out = []
    for n, d in streams:
        t = torch.linspace(0, 1, n, device=device) + torch.randn(B, n, generator=g, device=device) * 1e-3
        t = torch.sort(t, dim=1).values.contiguous()
        x = torch.randn(B, n, d, generator=g, device=device, dtype=torch.float32).to(dtype)
        out += [x, t]
    out.append(torch.linspace(0, 1, T, device=device).expand(B, -1).contiguous())
    return tuple(out)


def voxel_uniform_inputs(N=500_000, seed=0, device="cpu") -> torch.Tensor:
    """xyz ~ U[-10,10)^3; with grid_min -10, voxel 0.05, grid 128^3 only a corner lands in the grid."""
    g = _gen(seed, device)
    return torch.rand(N, 3, generator=g, device=device) * 20.0 - 10.0


def voxel_mixture_inputs(N=1 << 26, F=4, clusters=256, sigma=0.5, seed=0, device="cpu",
                         chunk=1 << 24, cluster_sorted=False) -> Tuple[torch.Tensor, torch.Tensor]:
    """Mixture of ``clusters`` isotropic Gaussians (centres U[-25,25)^3), F-channel N(0,1) features.
    Points come in iid order (the worst case for locality) unless ``cluster_sorted``, which emits the
    clusters one after another (a spatially coherent scan).  Generated in chunks so the peak temporary
    stays small."""
    g = _gen(seed, device)
    centres = torch.rand(clusters, 3, generator=g, device=device) * 50.0 - 25.0
    pts = torch.empty(N, 3, device=device)
    feats = torch.empty(N, F, device=device)
    for a in range(0, N, chunk):
        b = min(N, a + chunk)
        k = torch.randint(0, clusters, (b - a,), generator=g, device=device)
        if cluster_sorted:  # coherent within each generated chunk
            k = torch.sort(k).values
        pts[a:b] = centres[k] + sigma * torch.randn(b - a, 3, generator=g, device=device)
        feats[a:b] = torch.randn(b - a, F, generator=g, device=device)
    return pts, feats


VOXEL_OCCUPANCY_GEOMETRY = dict(grid_min=[-10.0, -10.0, -10.0], voxel_size=0.05, grid_size=[128, 128, 128])
VOXEL_MIXTURE_GEOMETRY = dict(grid_min=[-25.6, -25.6, -25.6], voxel_size=0.1, grid_size=[512, 512, 512])


# ----------------------------------------------------------------------------- byte accounting

def resample_bytes(B: int, S: int, T: int, D: int, elem: int) -> int:
    """Every input tensor once plus the output once (the reference's own formula:
    robocache/benchmarks/benchmark_trajectory_resample.cu:144-152)."""
    return B * S * D * elem + B * S * 4 + B * T * 4 + B * T * D * elem


def resample_touched_bytes(left: torch.Tensor, right: torch.Tensor, S: int, D: int, elem: int) -> int:
    """Bytes a kernel that skips unused source rows must still move: unique bracket rows + times + output."""
    B, T = left.shape
    base = torch.arange(B, device=left.device, dtype=torch.int64).unsqueeze(1) * S
    rows = torch.cat([(base + left.long()).flatten(), (base + right.long()).flatten()])
    touched = int(torch.unique(rows).numel())
    return touched * D * elem + B * S * 4 + B * T * 4 + B * T * D * elem


def fusion_bytes(B: int, T: int, elem: int, streams=FUSION_STREAMS) -> int:
    per = sum(n * d * elem + n * 4 for n, d in streams) + T * 4 + T * sum(d for _, d in streams) * elem
    return B * per


def voxel_bytes(N: int, F: int, grid_cells: int, mode: str, occupied: int = 0) -> Dict[str, int]:
    """Algorithmic bytes of one voxelisation call, zero-fill included."""
    pts = N * 12
    if mode in ("count", "occupancy"):
        return {"points": pts, "grid_zero_fill": grid_cells * 4, "total": pts + grid_cells * 4}
    feats = N * F * 4
    fill = grid_cells * 4 + grid_cells * F * 4
    norm = grid_cells * 4 + occupied * F * 4 * 2
    return {"points": pts + feats, "grid_zero_fill": fill, "normalize": norm, "total": pts + feats + fill + norm}
