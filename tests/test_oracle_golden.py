"""Pins the CPU oracle to the reference: golden vectors produced by the reference's own code
(tests/golden/make_golden.py) must be reproduced bit for bit."""
import pytest
import torch

import oracle
from conftest import bits, golden_names, load_golden


@pytest.mark.parametrize("name", golden_names("resample_"))
def test_resample_matches_reference_output(name):
    g = load_golden(name)
    out = oracle.resample_trajectories(g["src"], g["st"], g["tt"])
    assert out.shape == g["out"].shape
    assert torch.equal(bits(out), bits(g["out"])), name


@pytest.mark.parametrize("name", golden_names("resample_"))
def test_brackets_match_reference_indices(name):
    g = load_golden(name)
    left, right, w = oracle.brackets(g["st"], g["tt"])
    assert torch.equal(left, g["left"]) and torch.equal(right, g["right"])
    assert ((w >= 0) & (w <= 1)).all()


@pytest.mark.parametrize("name", golden_names("fusion_"))
def test_fusion_matches_reference_output(name):
    g = load_golden(name)
    out = oracle.fuse_multimodal(g["s1"], g["t1"], g["s2"], g["t2"], g["s3"], g["t3"], g["tt"])
    assert torch.equal(bits(out), bits(g["out"])), name


@pytest.mark.parametrize("name", golden_names("voxel_"))
def test_voxel_counts_match_reference_header(name):
    g = load_golden(name)
    gs = g["gs"].tolist()
    gmin = g["gmin"].tolist()
    vs = float(g["vs"])
    counts = oracle.voxelize_pointcloud(g["pts"], None, gmin, vs, gs, mode="count").flatten()
    occ = oracle.voxelize_pointcloud(g["pts"], None, gmin, vs, gs, mode="occupancy").flatten()
    nz = torch.nonzero(counts).flatten()
    assert torch.equal(nz, g["nz"])
    assert torch.equal(counts[nz].float(), g["density"])
    assert torch.equal(occ[nz].float(), g["occupancy"])
    assert int(occ.sum()) == nz.numel()


def test_known_answers_from_reference_tests():
    # robocache/tests/test_trajectory.py:55-71
    g = load_golden("resample_hand_ramp")
    out = oracle.resample_trajectories(g["src"], g["st"], g["tt"]).flatten()
    assert torch.allclose(out, torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0]), atol=1e-5)
    # robocache/python/robocache/__init__.py:391-397
    g = load_golden("resample_selftest")
    out = oracle.resample_trajectories(g["src"], g["st"], g["tt"]).flatten()
    assert torch.allclose(out, torch.tensor([1.5, 2.5]), atol=1e-4)
    # robocache/tests/test_all_operations.py:50-61 — one source row: every output equals it
    g = load_golden("resample_single_source")
    out = oracle.resample_trajectories(g["src"], g["st"], g["tt"])
    assert torch.allclose(out, g["src"].expand(-1, 5, -1), atol=1e-5)
    # robocache/tests/test_all_operations.py:63-75 — clamp outside the source range
    g = load_golden("resample_outside_range")
    out = oracle.resample_trajectories(g["src"], g["st"], g["tt"])
    assert torch.allclose(out[0, 0], g["src"][0, 0], atol=1e-5)
    assert torch.allclose(out[0, -1], g["src"][0, -1], atol=1e-5)
    # robocache/tests/test_voxelize_correctness.py:163-180 and :142-157
    g = load_golden("voxel_three_in_one")
    c = oracle.voxelize_pointcloud(g["pts"], None, g["gmin"].tolist(), float(g["vs"]), g["gs"].tolist(), "count")
    assert int(c.max()) == 3 and int(c.sum()) == 3
    g = load_golden("voxel_all_oob")
    c = oracle.voxelize_pointcloud(g["pts"], None, g["gmin"].tolist(), float(g["vs"]), g["gs"].tolist(), "count")
    assert int(c.sum()) == 0


def test_bf16_rounding_helper_matches_torch():
    x = torch.randn(10000) * torch.logspace(-20, 20, 10000)
    assert torch.equal(bits(oracle.round_to_bf16(x)), bits(x.bfloat16()))


def test_mean_mode_properties():
    g = torch.Generator().manual_seed(3)
    pts = torch.rand(5000, 3, generator=g) * 2 - 1
    feats = torch.randn(5000, 4, generator=g)
    grid, counts, sabs = oracle.voxelize_pointcloud(pts, feats, [-1, -1, -1], 0.25, [8, 8, 8], "mean", return_aux=True)
    ids = oracle.voxel_ids(pts, [-1, -1, -1], 0.25, [8, 8, 8])
    assert int(counts.sum()) == int((ids >= 0).sum())
    # weighted means recombine to the global feature sum of the in-grid points
    total = (grid * counts.unsqueeze(-1)).double().sum(dim=(0, 1, 2))
    assert torch.allclose(total, feats[ids >= 0].double().sum(0), atol=1e-3)
    assert (grid[counts == 0] == 0).all()


# ---- the torch restatement that bench.py times as the CPU baseline (oracle/torch_path.py)

@pytest.mark.parametrize("name", golden_names("resample_"))
def test_torch_path_resample_reproduces_reference_output(name):
    from oracle import torch_path
    g = load_golden(name)
    src = g["src"].float() if g["_bf16"] else g["src"]          # the fallback widens bf16 rows to fp32
    out = torch_path.interpolate_stream(g["src"], g["st"], g["tt"])
    assert torch.equal(bits(out.float()), bits(g["out"])), name
    assert torch.equal(bits(torch_path.interpolate_stream(src, g["st"], g["tt"])), bits(g["out"])), name


@pytest.mark.parametrize("name", golden_names("fusion_"))
def test_torch_path_fusion_reproduces_reference_output(name):
    from oracle import torch_path
    g = load_golden(name)
    out = torch_path.fuse_multimodal(g["s1"], g["t1"], g["s2"], g["t2"], g["s3"], g["t3"], g["tt"])
    assert torch.equal(bits(out.float()), bits(g["out"])), name


def test_torch_path_voxel_semantics_are_the_fallbacks_own():
    """Clamped, x-major: in-grid points agree with the oracle after a transpose, out-of-grid points land on the border."""
    from oracle import torch_path
    g = torch.Generator().manual_seed(8)
    pts = torch.rand(4000, 3, generator=g) * 1.8 - 0.9                  # all inside [-1, 1)^3
    kw = dict(grid_min=[-1.0, -1.0, -1.0], voxel_size=0.25, grid_size=[8, 8, 8])
    mine = oracle.voxelize_pointcloud(pts, None, mode="count", **kw)    # flat index vz*64 + vy*8 + vx
    theirs = torch_path.voxelize_pointcloud(pts, None, mode="count", **kw)   # indexed [vx][vy][vz]
    assert torch.equal(theirs, mine.reshape(8, 8, 8).permute(2, 1, 0))
    out = torch_path.voxelize_pointcloud(torch.tensor([[5.0, 0.0, 0.0]]), None, mode="occupancy", **kw)
    assert int(out.sum()) == 1 and int(out[7, 4, 4]) == 1
    feats = torch.randn(4000, 3, generator=g)
    m = torch_path.voxelize_pointcloud(pts, feats, mode="mean", **kw)
    om, oc, _ = oracle.voxelize_pointcloud(pts, feats, mode="mean", return_aux=True, **kw)
    assert torch.allclose(m, om.reshape(8, 8, 8, 3).permute(2, 1, 0, 3), atol=1e-5)
