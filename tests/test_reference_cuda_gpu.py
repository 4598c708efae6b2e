"""Second opinion from the reference's own CUDA kernels, compiled unmodified for sm_100a (oracle/_ref; skipped
where that library was not built).  The reference builds with --use_fast_math and, outside the source time
range, extrapolates where its torch path (the parity target) clamps, so values are compared with a tolerance
and only for targets inside the source range; voxel counts and occupancy must agree exactly for points that
are not within rounding distance of a voxel face (approximate division can move those)."""
import pytest
import torch

import oracle
import robocache
from robogoat_b200 import ops
import workloads

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(oracle.ref_cuda_lib() is None, reason="oracle/_ref CUDA library not built")]
DEV = "cuda:0"


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 2e-2)])
def test_resample_agrees_inside_the_source_range(dtype, tol):
    src, st, tt = (x.to(DEV) for x in workloads.resample_inputs(B=64, S=500, D=256, T=250, dtype=dtype,
                                                                 irregular_targets=True, seed=3))
    tt = tt.clamp(1e-4, 1 - 1e-4)                       # strictly inside [st[0], st[-1]] = [0, 1]
    ours = robocache.resample_trajectories(src, st, tt).float()
    ref = oracle.ref_cuda_resample(src, st, tt).float()
    torch.cuda.synchronize()
    assert (ours - ref).abs().max().item() <= tol * max(1.0, src.float().abs().max().item())


def test_fusion_agrees_inside_the_source_range():
    a = [x.to(DEV) for x in workloads.fusion_inputs(B=64, dtype=torch.float32, seed=4)]
    a[6] = a[6].clamp(0.02, 0.98).contiguous()          # jittered stream ends lie within 0.01 of 0 and 1
    ours = robocache.fuse_multimodal(*a)
    ref = oracle.ref_cuda_fuse(*a)
    torch.cuda.synchronize()
    assert (ours - ref).abs().max().item() <= 5e-5 * max(1.0, a[0].abs().max().item())


def test_voxel_counts_agree_away_from_voxel_faces():
    g = torch.Generator().manual_seed(6)
    kw = dict(grid_min=[-10.0, -10.0, -10.0], voxel_size=0.25, grid_size=[64, 64, 64])
    pts = torch.rand(200_000, 3, generator=g) * 20 - 10
    frac = ((pts + 10.0) / 0.25) % 1.0
    pts = pts[((frac > 1e-3) & (frac < 1 - 1e-3)).all(dim=1)].contiguous().to(DEV)
    feats = torch.randn(pts.shape[0], 4, generator=g).to(DEV)
    for mode in ("count", "occupancy"):
        ours = robocache.voxelize_pointcloud(pts, mode=mode, **kw)
        ref, _ = oracle.ref_cuda_voxelize(pts, None, kw["grid_min"], kw["voxel_size"], kw["grid_size"], mode)
        assert torch.equal(ours, ref), mode
    ours, counts = ops.voxelize_pointcloud_cuda(pts, feats, kw["grid_min"], kw["voxel_size"], kw["grid_size"], "mean")
    ref, rcounts = oracle.ref_cuda_voxelize(pts, feats, kw["grid_min"], kw["voxel_size"], kw["grid_size"], "mean")
    torch.cuda.synchronize()
    assert torch.equal(counts, rcounts)
    assert torch.allclose(ours, ref, rtol=1e-4, atol=1e-5)
