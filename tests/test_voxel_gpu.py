"""Parity of the CUDA voxeliser with the CPU oracle: occupancy and counts bit-exact, feature means
within |x-y| <= 1e-5*|y| + 1e-6*mean|f| (fp32 sums are order dependent)."""
import pytest
import torch

import oracle
import robocache
from conftest import golden_names, load_golden
from robogoat_b200 import ops
import workloads

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def dense_from_golden(g):
    V = int(g["gs"].prod())
    d = torch.zeros(V, dtype=torch.int32)
    d[g["nz"]] = g["density"].to(torch.int32)
    return d.view(*g["gs"].tolist())


@pytest.mark.parametrize("name", golden_names("voxel_"))
def test_golden_vectors(name, cuda_lib):
    g = load_golden(name)
    kw = dict(grid_min=g["gmin"].tolist(), voxel_size=float(g["vs"]), grid_size=g["gs"].tolist())
    exp = dense_from_golden(g)
    cnt = robocache.voxelize_pointcloud(g["pts"].to(DEV), mode="count", **kw)
    occ = robocache.voxelize_pointcloud(g["pts"].to(DEV), mode="occupancy", **kw)
    assert cnt.dtype == torch.int32 and occ.dtype == torch.int32      # robocache/tests/test_voxelize_correctness.py:128
    assert torch.equal(cnt.cpu(), exp)
    assert torch.equal(occ.cpu(), (exp > 0).int())


# sizes and grids of robocache/tests/test_voxelize_correctness.py:14-97 and test_voxel_optimized_correctness.py
@pytest.mark.parametrize("N", [0, 1, 3, 100, 127, 128, 129, 1000, 10_000, 500_000])
@pytest.mark.parametrize("G", [16, 32, 128])
def test_count_and_occupancy_exact(N, G, cuda_lib):
    g = torch.Generator().manual_seed(42 + N + G)
    pts = torch.rand(N, 3, generator=g) * 20 - 10
    kw = dict(grid_min=[-10.0, -10.0, -10.0], voxel_size=20.0 / G * 0.75, grid_size=[G, G, G])   # part of the cloud falls outside
    exp = oracle.voxelize_pointcloud(pts, None, mode="count", **kw)
    for agg in (False, True):
        cnt = ops.voxelize_pointcloud_cuda(pts.to(DEV), None, kw["grid_min"], kw["voxel_size"], kw["grid_size"], "count",
                                           warp_aggregate=agg)[0]
        assert torch.equal(cnt.cpu(), exp), f"agg={agg}"
    occ = robocache.voxelize_pointcloud(pts.to(DEV), mode="occupancy", **kw)
    assert torch.equal(occ.cpu(), (exp > 0).int())
    u8 = ops.voxelize_pointcloud_cuda(pts.to(DEV), None, kw["grid_min"], kw["voxel_size"], kw["grid_size"], "occupancy",
                                      occupancy_dtype=torch.uint8)[0]
    assert u8.dtype == torch.uint8 and torch.equal(u8.cpu().int(), (exp > 0).int())


def test_headline_occupancy_geometry(cuda_lib):
    """N=500000 in U[-10,10)^3 against a 128^3 grid of 0.05 m voxels at -10: most points are dropped."""
    pts = workloads.voxel_uniform_inputs(500_000, seed=0)
    kw = workloads.VOXEL_OCCUPANCY_GEOMETRY
    exp = oracle.voxelize_pointcloud(pts, None, mode="occupancy", **kw)
    occ = robocache.voxelize_pointcloud(pts.to(DEV), mode="occupancy", **kw)
    assert torch.equal(occ.cpu(), exp)
    assert 10_000 < int(exp.sum()) < 25_000
    occ2 = robocache.voxelize_occupancy(pts.to(DEV), torch.tensor(kw["grid_size"]), kw["voxel_size"], torch.tensor(kw["grid_min"]))
    assert torch.equal(occ2, occ)


def test_noncubic_layout_is_z_major(cuda_lib):
    pts = torch.tensor([[0.05, 0.15, 0.25]])            # voxel (0, 1, 2)
    out = robocache.voxelize_pointcloud(pts.to(DEV), grid_min=[0.0, 0.0, 0.0], voxel_size=0.1, grid_size=[4, 5, 6], mode="count")
    assert out.shape == (4, 5, 6)
    flat = out.flatten().cpu()
    assert int(flat[2 * 4 * 5 + 1 * 4 + 0]) == 1 and int(flat.sum()) == 1


def test_edge_points(cuda_lib):
    nan, inf = float("nan"), float("inf")
    pts = torch.tensor([[0.0, 0.0, 0.0], [-0.0, 0.0, 0.0], [-1e-7, 0.0, 0.0], [1.6, 0.0, 0.0], [1.5999999, 0.0, 0.0],
                        [nan, 0.0, 0.0], [inf, 0.0, 0.0], [-inf, 0.0, 0.0], [0.5, nan, 0.5], [1e30, 1e30, 1e30],
                        [0.3, 0.6, 0.9], [0.30000001, 0.6, 0.9]])
    kw = dict(grid_min=[0.0, 0.0, 0.0], voxel_size=0.1, grid_size=[16, 16, 16])
    exp = oracle.voxelize_pointcloud(pts, None, mode="count", **kw)
    out = robocache.voxelize_pointcloud(pts.to(DEV), mode="count", **kw)
    assert torch.equal(out.cpu(), exp)


def test_unaligned_points_view(cuda_lib):
    pts = workloads.voxel_uniform_inputs(1001, seed=1)
    kw = dict(grid_min=[-10.0, -10.0, -10.0], voxel_size=0.5, grid_size=[40, 40, 40])
    dev = pts.to(DEV)
    view = dev[1:]                                       # base pointer 12 bytes past a 16-byte boundary
    out = robocache.voxelize_pointcloud(view, mode="count", **kw)
    assert torch.equal(out.cpu(), oracle.voxelize_pointcloud(pts[1:], None, mode="count", **kw))


@pytest.mark.parametrize("F", [1, 2, 3, 4, 8, 6])
@pytest.mark.parametrize("N", [5, 1000, 200_000])
def test_mean_within_tolerance(F, N, cuda_lib):
    g = torch.Generator().manual_seed(F * 7 + N)
    pts = torch.rand(N, 3, generator=g) * 4 - 2
    feats = torch.randn(N, F, generator=g)
    kw = dict(grid_min=[-1.5, -1.5, -1.5], voxel_size=0.25, grid_size=[12, 12, 12])
    exp, ecnt, sabs = oracle.voxelize_pointcloud(pts, feats, mode="mean", return_aux=True, **kw)
    grid, counts = ops.voxelize_pointcloud_cuda(pts.to(DEV), feats.to(DEV), kw["grid_min"], kw["voxel_size"], kw["grid_size"], "mean")
    assert torch.equal(counts.cpu(), ecnt)
    tol = oracle.mean_tolerance(ecnt, sabs, exp)
    err = (grid.cpu() - exp).abs()
    assert bool((err <= tol).all()), f"max excess {(err - tol).max().item()}"
    assert bool((grid.cpu()[ecnt == 0] == 0).all())
    api = robocache.voxelize_pointcloud(pts.to(DEV), feats.to(DEV), mode="mean", **kw)
    assert api.shape == (12, 12, 12, F)
    # sums + separate normalisation over two slabs == fused call (the multi-GPU harness's split)
    sums, c2 = ops.voxelize_pointcloud_cuda(pts.to(DEV), feats.to(DEV), kw["grid_min"], kw["voxel_size"], kw["grid_size"], "mean", normalize=False)
    V = c2.numel()
    ops.voxel_normalize_cuda(sums, c2, 0, 701)
    ops.voxel_normalize_cuda(sums, c2, 701, V)
    assert bool(((sums.cpu() - exp).abs() <= tol).all())


def test_max_mode(cuda_lib):
    g = torch.Generator().manual_seed(5)
    pts = torch.rand(20_000, 3, generator=g) * 4 - 2
    feats = torch.randn(20_000, 3, generator=g)
    kw = dict(grid_min=[-1.5, -1.5, -1.5], voxel_size=0.25, grid_size=[12, 12, 12])
    ids = oracle.voxel_ids(pts, **kw)
    exp = torch.full((12 * 12 * 12, 3), float("-inf"))
    keep = ids >= 0
    exp.scatter_reduce_(0, ids[keep].unsqueeze(-1).expand(-1, 3), feats[keep], reduce="amax", include_self=True)
    exp = torch.where(torch.isfinite(exp), exp, torch.zeros_like(exp)).view(12, 12, 12, 3)
    out = robocache.voxelize_pointcloud(pts.to(DEV), feats.to(DEV), mode="max", **kw)
    assert torch.equal(out.cpu(), exp)


def test_errors(cuda_lib):
    pts = torch.zeros(10, 3, device=DEV)
    with pytest.raises(RuntimeError, match="Invalid mode"):
        robocache.voxelize_pointcloud(pts, mode="median")
    with pytest.raises(RuntimeError, match="features required"):
        robocache.voxelize_pointcloud(pts, mode="mean")
    with pytest.raises(RuntimeError, match="3 coordinates"):
        robocache.voxelize_pointcloud(torch.zeros(10, 4, device=DEV))
    with pytest.raises(RuntimeError, match="voxel_size must be positive"):
        robocache.voxelize_pointcloud(pts, voxel_size=0.0)
    with pytest.raises(RuntimeError, match="features must match"):
        robocache.voxelize_pointcloud(pts, torch.zeros(9, 2, device=DEV), mode="mean")
    with pytest.raises(RuntimeError, match="3 elements"):
        robocache.voxelize_pointcloud(pts, grid_size=[4, 4])


def test_guard_bands_and_determinism(cuda_lib):
    """Writes stay inside the grid (sentinel words either side, as
    robocache/tests/test_voxel_optimized_correctness.py:144-162) and integer outputs repeat exactly."""
    import ctypes
    L = cuda_lib
    pts = workloads.voxel_uniform_inputs(100_000, seed=3).to(DEV)
    G = 32
    V = G * G * G
    buf = torch.full((V + 512,), 0x5A5A5A5A, dtype=torch.int32, device=DEV)
    gmin = (ctypes.c_float * 3)(-10.0, -10.0, -10.0)
    gs = (ctypes.c_int32 * 3)(G, G, G)
    first = None
    for _ in range(5):                                   # robocache/tests/test_voxelize_correctness.py:188-230
        rc = L.rc_voxelize(pts.data_ptr(), None, buf.data_ptr() + 256 * 4, None, pts.shape[0], 0, gmin, 0.3, gs, 0, 1, 0,
                           torch.cuda.current_stream().cuda_stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert bool((buf[:256] == 0x5A5A5A5A).all()) and bool((buf[-256:] == 0x5A5A5A5A).all())
        cur = buf[256:-256].clone()
        first = cur if first is None else first
        assert torch.equal(cur, first)


def test_mixture_properties_at_scale(cuda_lib):
    """Count + mean on the headline cloud (2^26 mixture points, F=4, 512^3): counts
    sum to the in-grid points, means recombine to the global feature sums, empty voxels are exactly 0, and
    a 2^18 seeded prefix is checked voxel by voxel against the oracle on a sub-grid."""
    N = 1 << 26
    pts, feats = workloads.voxel_mixture_inputs(N, seed=0, device=DEV)
    kw = workloads.VOXEL_MIXTURE_GEOMETRY
    grid, counts = ops.voxelize_pointcloud_cuda(pts, feats, kw["grid_min"], kw["voxel_size"], kw["grid_size"], "mean")
    q = torch.floor((pts - torch.tensor(kw["grid_min"], device=DEV)) / torch.tensor(kw["voxel_size"], device=DEV))
    inside = ((q >= 0) & (q < 512)).all(dim=1)
    assert int(counts.sum(dtype=torch.int64)) == int(inside.sum())
    total = torch.stack([(grid[..., c].double() * counts).sum() for c in range(4)])
    ref_total = feats[inside].double().sum(0)
    assert torch.allclose(total, ref_total, rtol=1e-4, atol=1.0)
    assert bool((grid[counts == 0] == 0).all())
    cnt_only = robocache.voxelize_pointcloud(pts, mode="count", **kw)
    assert torch.equal(cnt_only, counts)
    del grid, q
    n = 1 << 18
    sub = dict(grid_min=kw["grid_min"], voxel_size=kw["voxel_size"], grid_size=[512, 512, 512])
    exp_ids = oracle.voxel_ids(pts[:n].cpu(), **sub)
    cnt_small = robocache.voxelize_pointcloud(pts[:n], mode="count", **kw).flatten()
    keep = exp_ids[exp_ids >= 0]
    exp_counts = torch.bincount(keep, minlength=512 ** 3).int()
    assert torch.equal(cnt_small.cpu(), exp_counts)


@pytest.mark.parametrize("cluster_sorted", [False, True])
def test_automatic_strategy_equals_single_pass(cluster_sorted, cuda_lib):
    """On grids larger than L2 the library probes the point order on the device and runs either one pass
    (coherent order) or slab passes / the two-phase id path (iid order).  Whatever it picks, counts must be
    identical to the forced single pass and means must agree within the summation-order tolerance."""
    N = 1 << 22
    pts, feats = workloads.voxel_mixture_inputs(N, seed=5, device=DEV, cluster_sorted=cluster_sorted)
    kw = workloads.VOXEL_MIXTURE_GEOMETRY
    args = (kw["grid_min"], kw["voxel_size"], kw["grid_size"])
    try:
        cuda_lib.rc_set_option(1, 1)
        ref_cnt = ops.voxelize_pointcloud_cuda(pts, None, *args, "count")[0]
        ref_mean, ref_c = ops.voxelize_pointcloud_cuda(pts, feats, *args, "mean")
        sabs, _ = ops.voxelize_pointcloud_cuda(pts, feats.abs(), *args, "mean", normalize=False)
        for forced in (0, 2, 5):
            cuda_lib.rc_set_option(1, forced)
            assert torch.equal(ops.voxelize_pointcloud_cuda(pts, None, *args, "count")[0], ref_cnt), forced
            mean, c = ops.voxelize_pointcloud_cuda(pts, feats, *args, "mean")
            assert torch.equal(c, ref_c), forced
            tol = 1e-5 * ref_mean.abs() + 1e-6 * sabs / ref_c.clamp(min=1).unsqueeze(-1)
            assert bool(((mean - ref_mean).abs() <= tol).all()), forced
    finally:
        cuda_lib.rc_set_option(1, 0)


@pytest.mark.parametrize("overlap,bulk", [(1, 1), (0, 1), (1, 0), (0, 0)])
@pytest.mark.parametrize("passes", [3, 16])
def test_run_path_switches_change_no_result(overlap, bulk, passes, cuda_lib):
    """Mean mode by slab-ordered runs with its launch and store forms switched: per-slab launches overlapped as
    programmatic dependents or ordinary, sorted chunks written by bulk asynchronous copies or by ordinary stores.
    Counts must equal the oracle's, means must lie within its tolerance, in every combination."""
    from robogoat_b200 import _lib
    N = 300_007
    pts, feats = workloads.voxel_mixture_inputs(N, seed=9)
    pts = pts * 0.25
    kw = dict(grid_min=[-6.4, -6.4, -6.4], voxel_size=0.1, grid_size=[128, 128, 128])
    exp, ecnt, sabs = oracle.voxelize_pointcloud(pts, feats, mode="mean", return_aux=True, **kw)
    cuda_lib.rc_set_option(_lib.OPT_VOXEL_PASSES, passes)
    cuda_lib.rc_set_option(_lib.OPT_SCATTER_OVERLAP, overlap)
    cuda_lib.rc_set_option(_lib.OPT_BUCKET_BULK_STORE, bulk)
    try:
        for _ in range(2):
            grid, counts = ops.voxelize_pointcloud_cuda(pts.to(DEV), feats.to(DEV), kw["grid_min"], kw["voxel_size"], kw["grid_size"], "mean")
            assert torch.equal(counts.cpu(), ecnt)
            assert bool(((grid.cpu() - exp).abs() <= oracle.mean_tolerance(ecnt, sabs, exp)).all())
    finally:
        cuda_lib.rc_set_option(_lib.OPT_VOXEL_PASSES, 0)
        cuda_lib.rc_set_option(_lib.OPT_SCATTER_OVERLAP, 1)
        cuda_lib.rc_set_option(_lib.OPT_BUCKET_BULK_STORE, 1)


def test_batched_float_grids_match_reference_header(cuda_lib):
    """[B,N,3] -> [B,D,H,W] float occupancy / density against the reference's own C++ header, item by item
    (skipped where that header was not compiled); also against the oracle, which is always available."""
    from robogoat_b200.batched import voxelize_density_batched, voxelize_occupancy_batched
    g = torch.Generator().manual_seed(17)
    B, N = 3, 5000
    pts = torch.rand(B, N, 3, generator=g) * 6 - 3
    origin, vs, dhw = [-2.0, -2.5, -1.0], 0.125, [20, 36, 28]          # depth(z), height(y), width(x)
    dens = voxelize_density_batched(pts.to(DEV), dhw, vs, origin).cpu()
    occ = voxelize_occupancy_batched(pts.to(DEV), torch.tensor(dhw), vs, torch.tensor(origin)).cpu()
    assert dens.shape == (B, 20, 36, 28) and dens.dtype == torch.float32
    for b in range(B):
        exp = oracle.voxelize_pointcloud(pts[b], None, origin, vs, [28, 36, 20], mode="count").flatten().float()
        assert torch.equal(dens[b].flatten(), exp)
        assert torch.equal(occ[b].flatten(), (exp > 0).float())
        ref = oracle.ref_header_voxelize(pts[b], origin, vs, [28, 36, 20], density=True)
        if ref is not None:
            assert torch.equal(dens[b].flatten(), ref)


@pytest.mark.parametrize("B,N", [(1, 1), (3, 5000), (5, 100), (64, 7), (2, 128), (4, 129), (2, 0)])
@pytest.mark.parametrize("F", [4, 3, 2])
def test_batched_one_launch_against_the_oracle_item_by_item(B, N, F, cuda_lib):
    """The batch kernel folds the item index into the voxel id; tiles of 128 points straddle items (N = 7, 100, 129),
    and every item must equal the single-cloud oracle: density and occupancy exact, feature means in tolerance,
    bounds exact (robocache/kernels/cutlass/point_cloud_voxelization.h:59-136, :218-227)."""
    from robogoat_b200.batched import (compute_point_cloud_bounds, voxelize_density_batched, voxelize_feature_max_batched,
                                       voxelize_feature_mean_batched, voxelize_occupancy_batched)
    g = torch.Generator().manual_seed(100 * B + N + F)
    pts = torch.rand(B, N, 3, generator=g) * 5 - 2.5
    feats = torch.randn(B, N, F, generator=g)
    origin, vs, dhw = [-2.0, -1.5, -1.0], 0.25, [9, 14, 17]            # depth(z), height(y), width(x)
    xyz = [17, 14, 9]
    dens = voxelize_density_batched(pts.to(DEV), dhw, vs, origin).cpu()
    occ = voxelize_occupancy_batched(pts.to(DEV), dhw, vs, origin).cpu()
    mean = voxelize_feature_mean_batched(pts.to(DEV), feats.to(DEV), dhw, vs, origin).cpu()
    fmax = voxelize_feature_max_batched(pts.to(DEV), feats.to(DEV), dhw, vs, origin).cpu()
    assert dens.shape == (B, 9, 14, 17) and mean.shape == (B, 9, 14, 17, F) and fmax.shape == mean.shape
    for b in range(B):
        exp = oracle.voxelize_pointcloud(pts[b], None, origin, vs, xyz, mode="count").flatten().float()
        assert torch.equal(dens[b].flatten(), exp), b
        assert torch.equal(occ[b].flatten(), (exp > 0).float()), b
        em, ec, sabs = oracle.voxelize_pointcloud(pts[b], feats[b], origin, vs, xyz, mode="mean", return_aux=True)
        tol = oracle.mean_tolerance(ec, sabs, em)
        assert bool(((mean[b].reshape(-1, F) - em.reshape(-1, F)).abs() <= tol.reshape(-1, F)).all()), b
        # feature max as the reference's kernel defines it: fmaxf against a zero-filled grid
        ids = oracle.voxel_ids(pts[b], origin, vs, xyz) if N else torch.empty(0, dtype=torch.int64)
        keep = ids >= 0
        want = torch.zeros(9 * 14 * 17, F)
        if int(keep.sum()):
            want.scatter_reduce_(0, ids[keep].unsqueeze(1).expand(-1, F), feats[b][keep], "amax", include_self=True)
        assert torch.equal(fmax[b].reshape(-1, F), want), b
    lo, hi = compute_point_cloud_bounds(pts.to(DEV))
    if N > 0:
        assert torch.equal(lo.cpu(), pts.amin(dim=1)) and torch.equal(hi.cpu(), pts.amax(dim=1))
    else:
        assert bool((lo == 1e10).all()) and bool((hi == -1e10).all())


@pytest.mark.gpu
@pytest.mark.parametrize("with_normals", [False, True])
@pytest.mark.parametrize("B,N", [(1, 1), (2, 300), (3, 45)])
def test_tsdf_matches_oracle(B, N, with_normals):
    """Truncated signed distances and weights, bit for bit against the CPU restatement of the reference's kernel rule
    (point_cloud_voxelization.cu:278-376): points inside, on the border of and outside the grid, a NaN point."""
    from oracle import tsdf as otsdf
    from robogoat_b200.batched import voxelize_tsdf
    g = torch.Generator().manual_seed(100 * B + N + int(with_normals))
    dhw, vs, origin, trunc = (12, 10, 14), 0.25, (-1.0, -0.5, -1.5), 0.6
    pts = torch.rand(B, N, 3, generator=g) * torch.tensor([4.5, 3.5, 4.0]) + torch.tensor([-1.5, -1.0, -2.0])
    if N > 10:
        pts[0, 3, 1] = float("nan")
        pts[-1, 5] = torch.tensor([1e30, 0.0, 0.0])
        pts[0, 7] = torch.tensor([-1.0 + 0.125, -0.5 + 0.125, -1.5 + 0.125])     # exactly on a voxel centre
    nrm = None
    if with_normals:
        nrm = torch.randn(B, N, 3, generator=g)
        nrm = nrm / nrm.norm(dim=2, keepdim=True)
    t, w = voxelize_tsdf(pts.to(DEV), nrm.to(DEV) if nrm is not None else None, dhw, vs, origin, trunc)
    et, ew = otsdf.voxelize_tsdf(pts.numpy(), nrm.numpy() if nrm is not None else None, dhw, vs, origin, trunc)
    assert t.shape == (B, *dhw) and w.shape == (B, *dhw)
    assert torch.equal(w.cpu(), torch.from_numpy(ew))
    assert torch.equal(t.cpu().view(torch.int32), torch.from_numpy(et).view(torch.int32))
    assert N <= 10 or float(ew.sum()) > 0


@pytest.mark.gpu
def test_tsdf_neighbourhood_larger_than_2_pow_20_cells():
    """A truncation distance that covers the whole grid of 1.155 M voxels: neighbourhoods above 2^20 cells index their
    cells by division instead of the reciprocal multiply."""
    from oracle import tsdf as otsdf
    from robogoat_b200.batched import voxelize_tsdf
    dhw, vs, origin, trunc = (100, 105, 110), 1.0, (0.0, 0.0, 0.0), 200.0
    pts = torch.tensor([[[3.2, 50.1, 97.7], [60.5, 10.25, 20.0], [109.9, 104.9, 0.1]]])
    nrm = torch.tensor([[[1.0, 0.0, 0.0], [0.0, -1.0, 0.0], [0.6, 0.0, 0.8]]])
    t, w = voxelize_tsdf(pts.to(DEV), nrm.to(DEV), dhw, vs, origin, trunc)
    et, ew = otsdf.voxelize_tsdf(pts.numpy(), nrm.numpy(), dhw, vs, origin, trunc)
    assert torch.equal(w.cpu(), torch.from_numpy(ew)) and float(ew.min()) == 3.0
    assert torch.equal(t.cpu().view(torch.int32), torch.from_numpy(et).view(torch.int32))


@pytest.mark.gpu
def test_tsdf_argument_errors_and_empty():
    from robogoat_b200.batched import voxelize_tsdf
    pts = torch.zeros(1, 4, 3, device=DEV)
    with pytest.raises(RuntimeError):
        voxelize_tsdf(pts, None, (4, 4, 4), 0.1, (0, 0, 0), 0.0)            # truncation must be positive
    with pytest.raises(RuntimeError):
        voxelize_tsdf(pts, None, (4, 4, 4), 0.001, (0, 0, 0), 10.0)         # neighbourhood beyond the supported reach
    with pytest.raises(ValueError):
        voxelize_tsdf(pts, torch.zeros(1, 3, 3, device=DEV), (4, 4, 4), 0.1, (0, 0, 0), 0.2)
    t, w = voxelize_tsdf(torch.zeros(2, 0, 3, device=DEV), None, (3, 3, 3), 0.1, (0, 0, 0), 0.2)
    assert float(t.abs().sum()) == 0 and float(w.sum()) == 0
