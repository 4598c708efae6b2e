"""Randomised shape sweep of the interpolation kernels against the oracle: stream counts, lengths, widths
and batch sizes are drawn from a seeded generator so that every access width (16/8/4/2 bytes), both kernels
(row-gather and TMA-staged block, 8- and 16-byte output paths) and their tile/edge handling are hit by shapes
nobody hand-picked.  Every case is bit-exact (see test_resample_gpu.py for the gates)."""
import random

import pytest
import torch

import oracle
from robogoat_b200 import ops
import workloads
from test_resample_gpu import DEV, assert_exact

pytestmark = [pytest.mark.gpu, pytest.mark.usefixtures("kernel_choice")]


def _case(seed):
    rnd = random.Random(seed)
    ns = rnd.choice([1, 1, 2, 3, 3, 4])
    B = rnd.choice([1, 2, 3, 5, 17, 40, 300])
    T = rnd.choice([1, 2, 7, 31, 32, 33, 50, 129, 250])
    dtype = rnd.choice([torch.float32, torch.bfloat16])
    widths = [rnd.choice([1, 2, 3, 4, 6, 8, 12, 16, 20, 64, 100, 128, 256, 512]) for _ in range(ns)]
    lens = [rnd.choice([1, 2, 3, 10, 30, 100, 200, 333]) for _ in range(ns)]
    return ns, B, T, dtype, widths, lens


@pytest.mark.parametrize("seed", range(40))
def test_random_shapes(seed, cuda_lib):
    ns, B, T, dtype, widths, lens = _case(seed)
    g = torch.Generator().manual_seed(1000 + seed)
    datas, times = [], []
    for n, d in zip(lens, widths):
        datas.append(torch.randn(B, n, d, generator=g).to(dtype))
        times.append(workloads.cumsum_times(B, n, g))
    tt = torch.rand(B, T, generator=g) * 1.3 - 0.15
    got = ops.fuse_streams_cuda([d.to(DEV) for d in datas], [t.to(DEV) for t in times], tt.to(DEV)).cpu()
    parts = [oracle.resample_trajectories(d, t, tt) for d, t in zip(datas, times)]
    exp = torch.cat(parts, dim=-1)
    if dtype == torch.bfloat16:
        exp = oracle.round_to_bf16(exp)
    assert_exact(got, exp, f"seed {seed}: ns={ns} B={B} T={T} {dtype} widths={widths} lens={lens}")


@pytest.mark.parametrize("seed", range(24))
def test_random_voxel_geometries(seed, cuda_lib):
    """Random grids (non-cubic, odd sizes), voxel sizes, cloud sizes and feature widths: counts and occupancy
    exact, means within the summation-order tolerance, max exact."""
    import robocache
    rnd = random.Random(500 + seed)
    gs = [rnd.choice([1, 3, 8, 17, 32, 50, 96]) for _ in range(3)]
    vs = rnd.choice([0.05, 0.1, 0.13, 0.25, 1.0])
    gmin = [rnd.uniform(-5, 5) for _ in range(3)]
    N = rnd.choice([1, 31, 128, 1000, 4097, 60_000])
    F = rnd.choice([1, 2, 3, 4, 5, 8])
    g = torch.Generator().manual_seed(seed)
    span = torch.tensor([gs[0] * vs, gs[1] * vs, gs[2] * vs])
    pts = torch.rand(N, 3, generator=g) * span * 1.3 + torch.tensor(gmin) - 0.15 * span   # part of the cloud falls outside
    feats = torch.randn(N, F, generator=g)
    kw = dict(grid_min=gmin, voxel_size=vs, grid_size=gs)
    exp_cnt = oracle.voxelize_pointcloud(pts, None, mode="count", **kw)
    assert torch.equal(robocache.voxelize_pointcloud(pts.to(DEV), mode="count", **kw).cpu(), exp_cnt), (seed, gs, vs, N)
    assert torch.equal(robocache.voxelize_pointcloud(pts.to(DEV), mode="occupancy", **kw).cpu(), (exp_cnt > 0).int())
    exp, ecnt, sabs = oracle.voxelize_pointcloud(pts, feats, mode="mean", return_aux=True, **kw)
    got = robocache.voxelize_pointcloud(pts.to(DEV), feats.to(DEV), mode="mean", **kw).cpu()
    assert bool(((got - exp).abs() <= oracle.mean_tolerance(ecnt, sabs, exp)).all()), (seed, gs, vs, N, F)
    ids = oracle.voxel_ids(pts, **kw)
    V = gs[0] * gs[1] * gs[2]
    mx = torch.full((V, F), float("-inf"))
    keep = ids >= 0
    if bool(keep.any()):
        mx.scatter_reduce_(0, ids[keep].unsqueeze(-1).expand(-1, F), feats[keep], reduce="amax", include_self=True)
    mx = torch.where(torch.isfinite(mx), mx, torch.zeros_like(mx)).view(gs[0], gs[1], gs[2], F)
    assert torch.equal(robocache.voxelize_pointcloud(pts.to(DEV), feats.to(DEV), mode="max", **kw).cpu(), mx)
