"""The two kernels of the multi-GPU point exchange, checked on one GPU: the stable partition of a cloud by
owning slab against a stable sort of the oracle's voxel ids, and the id scatter of every bucket into its slab
against the single-call grid."""
import pytest
import torch

import oracle
from robogoat_b200 import ops, sharding

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _cloud(N, seed, F=4):
    g = torch.Generator().manual_seed(seed)
    pts = torch.rand(N, 3, generator=g) * 5 - 2.5            # part of it falls outside the grid
    if N > 10:
        pts[3] = float("nan")
        pts[7, 1] = float("inf")
    return pts, torch.randn(N, F, generator=g)


@pytest.mark.parametrize("N", [0, 1, 127, 128, 1000, 33_333, 300_001])
@pytest.mark.parametrize("parts", [1, 2, 3, 8, 64])
def test_partition_is_the_stable_sort_by_owner(N, parts, cuda_lib):
    kw = dict(grid_min=[-2.0, -2.0, -2.0], voxel_size=0.25, grid_size=[16, 15, 13])
    V = 16 * 15 * 13
    pts, feats = _cloud(N, 100 + parts)
    ids, fb, pc = ops.voxel_partition_cuda(pts.to(DEV), feats.to(DEV), kw["grid_min"], kw["voxel_size"], kw["grid_size"], parts)
    exp_ids = oracle.voxel_ids(pts, **kw) if N else torch.empty(0, dtype=torch.int64)
    keep = exp_ids >= 0
    per = (V + parts - 1) // parts
    owner = exp_ids[keep] // per
    order = torch.sort(owner, stable=True).indices
    n = int(keep.sum())
    assert pc.cpu().tolist() == torch.bincount(owner, minlength=parts).tolist()
    assert torch.equal(ids[:n].cpu().long(), exp_ids[keep][order])
    assert torch.equal(fb[:n].cpu(), feats[keep][order])


def _owner(ids, V, groups, per_group):
    slab = (V + groups - 1) // groups
    sub = (slab + per_group - 1) // per_group
    grp = ids // slab
    return grp * per_group + (ids - grp * slab) // sub


@pytest.mark.parametrize("groups,per_group", [(1, 7), (2, 3), (3, 5), (8, 4), (2, 32), (8, 8)])
@pytest.mark.parametrize("N", [1000, 70_001])
def test_two_level_partition_and_run_scatter(groups, per_group, N, cuda_lib):
    """Sub-ranges inside every owner's slab: the partition is still the stable sort by part, and scattering the
    runs of every owner, one pass per sub-range, rebuilds that owner's slab."""
    import robocache
    kw = dict(grid_min=[-2.0, -2.0, -2.0], voxel_size=0.25, grid_size=[16, 15, 13])
    V = 16 * 15 * 13
    pts, feats = _cloud(N, 31 * groups + per_group)
    p, f = pts.to(DEV), feats.to(DEV)
    ids, fb, pc = ops.voxel_partition_cuda(p, f, kw["grid_min"], kw["voxel_size"], kw["grid_size"], groups, per_group)
    exp_ids = oracle.voxel_ids(pts, **kw)
    keep = exp_ids >= 0
    owner = _owner(exp_ids[keep], V, groups, per_group)
    order = torch.sort(owner, stable=True).indices
    n = int(keep.sum())
    counts = pc.cpu().tolist()
    assert counts == torch.bincount(owner, minlength=groups * per_group).tolist()
    assert torch.equal(ids[:n].cpu().long(), exp_ids[keep][order])
    assert torch.equal(fb[:n].cpu(), feats[keep][order])
    starts = [0]
    for c in counts:
        starts.append(starts[-1] + c)
    full_cnt = robocache.voxelize_pointcloud(p, mode="count", **kw).reshape(V)
    exp, ecnt, sabs = oracle.voxelize_pointcloud(pts, feats, mode="mean", return_aux=True, **kw)
    tol = oracle.mean_tolerance(ecnt, sabs, exp).reshape(V, 4)
    for g in range(groups):
        a, b = sharding.slab_bounds(V, g, groups)
        runs = [(starts[g * per_group + k], counts[g * per_group + k], k) for k in range(per_group)]
        got = ops.voxel_scatter_runs_cuda(ids.data_ptr(), None, p.device, 0, a, b, runs, per_group, "count")[0]
        assert torch.equal(got, full_cnt[a:b])
        got = ops.voxel_scatter_runs_cuda(ids.data_ptr(), None, p.device, 0, a, b, runs, per_group, "occupancy")[0]
        assert torch.equal(got, (full_cnt[a:b] > 0).int())
        grid, cnt = ops.voxel_scatter_runs_cuda(ids.data_ptr(), fb.data_ptr(), p.device, 4, a, b, runs, per_group, "mean")
        assert torch.equal(cnt, full_cnt[a:b])
        assert bool(((grid.cpu() - exp.reshape(V, 4)[a:b]).abs() <= tol[a:b]).all())
        bufs = ops.voxel_slab_buffers(b - a, 4, "mean", p.device)          # accumulators cleared by the caller
        for t in bufs:
            t.zero_()
        grid2, cnt2 = ops.voxel_scatter_runs_cuda(ids.data_ptr(), fb.data_ptr(), p.device, 4, a, b, runs, per_group, "mean", out=bufs)
        assert grid2.data_ptr() == bufs[0].data_ptr() and torch.equal(cnt2, cnt)
        assert bool(((grid2.cpu() - exp.reshape(V, 4)[a:b]).abs() <= tol[a:b]).all())


@pytest.mark.parametrize("remote", [False, True])      # True: the line-aligned store path, here with start slots off the line
@pytest.mark.parametrize("N", [50_000, 6_000_000])
def test_split_count_and_move_into_separate_destinations(remote, N, cuda_lib):
    """The two halves called separately, every part into a buffer of its own at a chosen slot - the form the
    direct exchange uses with peer buffers."""
    kw = dict(grid_min=[-2.0, -2.0, -2.0], voxel_size=0.25, grid_size=[16, 16, 16])
    V = 16 ** 3
    pts, feats = _cloud(N, 5)
    p, f = pts.to(DEV), feats.to(DEV)
    groups, per_group = 2, 3
    pc, scratch = ops.voxel_partition_count_cuda(p, kw["grid_min"], kw["voxel_size"], kw["grid_size"], groups, per_group)
    counts = pc.tolist()
    exp_ids = oracle.voxel_ids(pts, **kw)
    keep = exp_ids >= 0
    owner = _owner(exp_ids[keep], V, groups, per_group)
    assert counts == torch.bincount(owner, minlength=6).tolist()
    pad = 5
    bufs_i = [torch.full((c + 2 * pad,), -7, dtype=torch.int32, device=DEV) for c in counts]
    bufs_f = [torch.full((c + 2 * pad, 4), -7.0, device=DEV) for c in counts]
    ops.voxel_partition_move_cuda(p, f, kw["grid_min"], kw["voxel_size"], kw["grid_size"], groups, per_group,
                                  [t.data_ptr() for t in bufs_i], [t.data_ptr() for t in bufs_f], [pad] * 6, scratch, remote=remote)
    for part in range(6):
        sel = owner == part
        assert torch.equal(bufs_i[part][pad:pad + counts[part]].cpu().long(), exp_ids[keep][sel])
        assert torch.equal(bufs_f[part][pad:pad + counts[part]].cpu(), feats[keep][sel])
        assert bool((bufs_i[part][:pad] == -7).all()) and bool((bufs_i[part][pad + counts[part]:] == -7).all())   # guard bands
        assert bool((bufs_f[part][:pad] == -7).all()) and bool((bufs_f[part][pad + counts[part]:] == -7).all())


@pytest.mark.parametrize("F", [1, 2, 3, 4, 8])
def test_partition_moves_feature_rows_of_any_width(F, cuda_lib):
    kw = dict(grid_min=[-2.0, -2.0, -2.0], voxel_size=0.5, grid_size=[8, 8, 8])
    pts, feats = _cloud(5000, F, F=F)
    ids, fb, pc = ops.voxel_partition_cuda(pts.to(DEV), feats.to(DEV), kw["grid_min"], kw["voxel_size"], kw["grid_size"], 4)
    exp_ids = oracle.voxel_ids(pts, **kw)
    keep = exp_ids >= 0
    order = torch.sort(exp_ids[keep] // 128, stable=True).indices
    n = int(keep.sum())
    assert int(pc.sum()) == n and torch.equal(fb[:n].cpu(), feats[keep][order])
    ids2, none, pc2 = ops.voxel_partition_cuda(pts.to(DEV), None, kw["grid_min"], kw["voxel_size"], kw["grid_size"], 4)
    assert none is None and torch.equal(ids2[:n], ids[:n]) and torch.equal(pc, pc2)


@pytest.mark.parametrize("parts", [1, 2, 5, 8])
def test_buckets_scattered_into_their_slabs_rebuild_the_grid(parts, cuda_lib):
    import robocache
    kw = dict(grid_min=[-2.0, -2.0, -2.0], voxel_size=0.125, grid_size=[32, 31, 30])
    V = 32 * 31 * 30
    pts, feats = _cloud(200_000, 7)
    p, f = pts.to(DEV), feats.to(DEV)
    ids, fb, pc = ops.voxel_partition_cuda(p, f, kw["grid_min"], kw["voxel_size"], kw["grid_size"], parts)
    starts = [0]
    for c in pc.tolist():
        starts.append(starts[-1] + c)
    full_cnt = robocache.voxelize_pointcloud(p, mode="count", **kw).reshape(V)
    full_occ = robocache.voxelize_pointcloud(p, mode="occupancy", **kw).reshape(V)
    exp, ecnt, sabs = oracle.voxelize_pointcloud(pts, feats, mode="mean", return_aux=True, **kw)
    tol = oracle.mean_tolerance(ecnt, sabs, exp).reshape(V, 4)
    for r in range(parts):
        a, b = sharding.slab_bounds(V, r, parts)
        # every rank sees all buckets here; ids outside its slab must be ignored, so hand it the whole list too
        for lo, hi in ((starts[r], starts[r + 1]), (0, starts[-1])):
            if lo % 4:                                   # the id list must start on a 16-byte boundary
                my_ids, my_f = ids[lo:hi].clone(), fb[lo:hi].clone()
            else:
                my_ids, my_f = ids[lo:hi], fb[lo:hi]
            assert torch.equal(ops.voxel_scatter_ids_cuda(my_ids, None, a, b, "count")[0], full_cnt[a:b])
            assert torch.equal(ops.voxel_scatter_ids_cuda(my_ids, None, a, b, "occupancy")[0], full_occ[a:b])
            grid, cnt = ops.voxel_scatter_ids_cuda(my_ids, my_f, a, b, "mean")
            assert torch.equal(cnt, full_cnt[a:b])
            assert bool(((grid.cpu() - exp.reshape(V, 4)[a:b]).abs() <= tol[a:b]).all())


def test_scatter_ids_slab_passes_agree(cuda_lib):
    """Forcing several slab passes must not change counts, and leaves means within the summation-order tolerance."""
    from robogoat_b200 import _lib
    kw = dict(grid_min=[-2.0, -2.0, -2.0], voxel_size=0.125, grid_size=[32, 32, 32])
    pts, feats = _cloud(100_000, 11)
    ids, fb, pc = ops.voxel_partition_cuda(pts.to(DEV), feats.to(DEV), kw["grid_min"], kw["voxel_size"], kw["grid_size"], 1)
    n = int(pc.sum())
    one = ops.voxel_scatter_ids_cuda(ids[:n], fb[:n], 0, 32 ** 3, "mean")
    L = _lib.load()
    try:
        assert L.rc_set_option(1, 5) == 0
        five = ops.voxel_scatter_ids_cuda(ids[:n], fb[:n], 0, 32 ** 3, "mean")
    finally:
        L.rc_set_option(1, 0)
    assert torch.equal(one[1], five[1])
    assert torch.allclose(one[0], five[0], rtol=1e-5, atol=1e-6)


def test_exchange_entry_points_reject_bad_arguments(cuda_lib):
    pts = torch.zeros(10, 3, device=DEV)
    with pytest.raises(RuntimeError):
        ops.voxel_partition_cuda(pts, None, [0, 0, 0], 0.1, [4, 4, 4], 65)
    with pytest.raises(RuntimeError):
        ops.voxel_scatter_ids_cuda(torch.zeros(4, dtype=torch.int32, device=DEV), None, 0, 8, "max")
    with pytest.raises(RuntimeError):
        ops.voxel_scatter_ids_cuda(torch.zeros(8, dtype=torch.int32, device=DEV)[1:5], None, 0, 8, "count")  # misaligned ids


@pytest.mark.parametrize("groups,per_group", [(1, 1), (2, 1), (8, 4), (4, 16), (2, 14), (8, 8)])
@pytest.mark.parametrize("N", [150_001, 7_000_003])      # the larger cloud gives every CTA several chunks: records wait across chunks
def test_line_aligned_and_plain_stores_write_the_same_bytes(groups, per_group, N, cuda_lib):
    from robogoat_b200 import _lib
    kw = dict(grid_min=[-2.0, -2.0, -2.0], voxel_size=0.125, grid_size=[32, 32, 32])
    pts, feats = _cloud(N, 77)
    p, f = pts.to(DEV), feats.to(DEV)
    L = _lib.load()
    outs = []
    try:
        for aligned in (2, 0):
            assert L.rc_set_option(2, aligned) == 0
            ids, fb, pc = ops.voxel_partition_cuda(p, f, kw["grid_min"], kw["voxel_size"], kw["grid_size"], groups, per_group)
            n = int(pc.sum())
            outs.append((ids[:n].clone(), fb[:n].clone(), pc.clone()))
    finally:
        L.rc_set_option(2, 1)
    assert torch.equal(outs[0][2], outs[1][2]) and torch.equal(outs[0][0], outs[1][0])
    assert torch.equal(outs[0][1], outs[1][1])
    exp_ids = oracle.voxel_ids(pts, **kw)
    keep = exp_ids >= 0
    order = torch.sort(_owner(exp_ids[keep], 32 ** 3, groups, per_group), stable=True).indices
    assert torch.equal(outs[0][1].cpu(), feats[keep][order])


@pytest.fixture(params=["bulk-stores", "plain-stores"])
def bucket_store_choice(request, cuda_lib):
    """The bucket kernel's write-out by bulk asynchronous copies (the default) and by ordinary stores: same bytes."""
    from robogoat_b200 import _lib
    cuda_lib.rc_set_option(_lib.OPT_BUCKET_BULK_STORE, 1 if request.param == "bulk-stores" else 0)
    yield request.param
    cuda_lib.rc_set_option(_lib.OPT_BUCKET_BULK_STORE, 1)


@pytest.mark.parametrize("layout", ["owner-pools", "source-pools"])
@pytest.mark.parametrize("R,K", [(1, 1), (2, 8), (3, 2), (4, 4), (8, 2), (16, 1)])
@pytest.mark.parametrize("N", [0, 1, 2500, 40_001])
def test_bucket_exchange_with_every_rank_on_one_gpu(R, K, N, layout, bucket_store_choice, cuda_lib):
    """The bucket form of the exchange with all ranks' pools in this GPU's memory, in both layouts: "owner-pools" (every
    source stores into the owners' pools, block source * chunks + chunk; an owner reads its one pool) and "source-pools"
    (every source fills a region per owner of its own pool; an owner reads its region of every source's pool).  Each
    slab must equal the oracle's grid of the whole cloud.  The pools start out full of garbage: whatever a source does
    not write must not be read.  The shards are uneven and one more chunk than needed is reserved per source."""
    kw = dict(grid_min=[-2.0, -2.0, -2.0], voxel_size=0.25, grid_size=[16, 15, 13])       # 3120 voxels: not a multiple of 16
    V = 16 * 15 * 13
    pts, feats = _cloud(N, 500 + R * K + N)
    cuts = [0] + sorted(torch.randint(0, N + 1, (R - 1,), generator=torch.Generator().manual_seed(R + N)).tolist()) + [N]
    chunks = (max(b - a for a, b in zip(cuts, cuts[1:])) + 1023) // 1024 + 1
    blk = int(cuda_lib.rc_voxel_bucket_block_records(K))
    assert blk % 32 == 0 and blk >= 1024 + 8 * K
    nblocks = R * chunks
    # R pools of R * chunks blocks: pool d belongs to owner d ("owner-pools") or to source d ("source-pools")
    pools = [dict(ids=torch.full((nblocks * blk,), 123456789, dtype=torch.int32, device=DEV),
                  feats=torch.full((nblocks * blk, 4), float("nan"), device=DEV),
                  runs=torch.full((K * nblocks,), 0x7fff7fff, dtype=torch.int32, device=DEV)) for _ in range(R)]
    rec = chunks * blk
    for s in range(R):
        a, b = cuts[s], cuts[s + 1]
        if layout == "owner-pools":
            dest = ([p["ids"].data_ptr() for p in pools], [p["feats"].data_ptr() for p in pools],
                    [p["runs"].data_ptr() for p in pools], s * chunks, nblocks)
        else:
            me = pools[s]
            dest = ([me["ids"].data_ptr() + d * rec * 4 for d in range(R)], [me["feats"].data_ptr() + d * rec * 16 for d in range(R)],
                    [me["runs"].data_ptr() + d * K * chunks * 4 for d in range(R)], 0, chunks)
        ops.voxel_bucket_exchange_cuda(pts[a:b].to(DEV), feats[a:b].to(DEV), kw["grid_min"], kw["voxel_size"], kw["grid_size"],
                                       R, K, chunks, dest[3], dest[4], dest[0], dest[1], dest[2])
    if N:
        exp, ecnt, sabs = oracle.voxelize_pointcloud(pts, feats, mode="mean", return_aux=True, **kw)
        tol = oracle.mean_tolerance(ecnt, sabs, exp).reshape(V, 4)
        exp, ecnt = exp.reshape(V, 4), ecnt.reshape(V)
    else:
        exp, ecnt, tol = torch.zeros(V, 4), torch.zeros(V, dtype=torch.int32), torch.zeros(V, 4)
    total = 0
    for d in range(R):
        lo, hi = sharding.slab_bounds(V, d, R)
        if layout == "owner-pools":
            src = ([pools[d]["ids"].data_ptr()], [pools[d]["feats"].data_ptr()], [pools[d]["runs"].data_ptr()], nblocks)
        else:
            src = ([p["ids"].data_ptr() + d * rec * 4 for p in pools], [p["feats"].data_ptr() + d * rec * 16 for p in pools],
                   [p["runs"].data_ptr() + d * K * chunks * 4 for p in pools], chunks)
        grid, counts = ops.voxel_scatter_buckets_cuda(src[0], src[1], src[2], src[3], K, DEV, lo, hi)
        assert torch.equal(counts.cpu(), ecnt[lo:hi]), (d, R, K)
        assert bool(((grid.cpu() - exp[lo:hi]).abs() <= tol[lo:hi]).all()), (d, R, K)
        total += int(counts.sum())
    assert total == int(ecnt.sum())
    torch.cuda.synchronize()


@pytest.mark.gpu
@pytest.mark.parametrize("R,K,slices", [(2, 4, 3), (4, 2, 4), (3, 1, 2)])
def test_bucket_exchange_in_slices_on_one_gpu(R, K, slices, cuda_lib):
    """The sliced form's calls with every rank on this GPU: each source buckets its cloud slice by slice (a small grid
    per launch), each owner clears its slab with a source-less call, accumulates slice after slice from windows of its
    pool (one window per source, run tables addressed with the pool's row length) without clearing, and normalises
    with the last slice.  Every slab must equal the oracle's grid of the whole cloud."""
    kw = dict(grid_min=[-2.0, -2.0, -2.0], voxel_size=0.25, grid_size=[16, 15, 13])
    V = 16 * 15 * 13
    N = 30_000
    pts, feats = _cloud(N, 900 + R + K)
    cuts = [N * r // R for r in range(R + 1)]
    chunks = (N // R + 1023) // 1024 + 2            # capacity per source; the last slice of some sources stays empty
    cs = (chunks + slices - 1) // slices
    blk = int(cuda_lib.rc_voxel_bucket_block_records(K))
    nblocks = R * chunks
    pools = [dict(ids=torch.full((nblocks * blk,), 123456789, dtype=torch.int32, device=DEV),
                  feats=torch.full((nblocks * blk, 4), float("nan"), device=DEV),
                  runs=torch.full((K * nblocks,), 0x7fff7fff, dtype=torch.int32, device=DEV)) for _ in range(R)]
    dest = ([p["ids"].data_ptr() for p in pools], [p["feats"].data_ptr() for p in pools], [p["runs"].data_ptr() for p in pools])
    for r in range(R):
        p_r, f_r = pts[cuts[r]:cuts[r + 1]].to(DEV), feats[cuts[r]:cuts[r + 1]].to(DEV)
        n_r = p_r.shape[0]
        for s in range(slices):
            c0 = min(s * cs, chunks)
            nch = min(cs, chunks - c0)
            p0, p1 = min(n_r, c0 * 1024), min(n_r, (c0 + nch) * 1024)
            ops.voxel_bucket_exchange_cuda(p_r[p0:p1], f_r[p0:p1], kw["grid_min"], kw["voxel_size"], kw["grid_size"], R, K, nch,
                                           r * chunks + c0, nblocks, *dest, ctas_per_sm=1 + s % 3)
    exp, ecnt, sabs = oracle.voxelize_pointcloud(pts, feats, mode="mean", return_aux=True, **kw)
    tol = oracle.mean_tolerance(ecnt, sabs, exp).reshape(V, 4)
    exp, ecnt = exp.reshape(V, 4), ecnt.reshape(V)
    for d in range(R):
        lo, hi = sharding.slab_bounds(V, d, R)
        out = ops.voxel_slab_buffers(hi - lo, 4, "mean", torch.device(DEV))
        out[0].fill_(float("nan")); out[1].fill_(77)
        ops.voxel_scatter_buckets_cuda([], [], [], 0, K, DEV, lo, hi, normalize=False, out=out)      # clears only
        assert int(out[1].abs().sum()) == 0 and float(out[0].abs().sum()) == 0.0
        for s in range(slices):
            c0 = min(s * cs, chunks)
            nch = min(cs, chunks - c0)
            first = [r * chunks + c0 for r in range(R)]
            ops.voxel_scatter_buckets_cuda([pools[d]["ids"].data_ptr() + b * blk * 4 for b in first],
                                           [pools[d]["feats"].data_ptr() + b * blk * 16 for b in first],
                                           [pools[d]["runs"].data_ptr() + b * 4 for b in first], nch, K, DEV, lo, hi,
                                           normalize=(s == slices - 1), table_row_blocks=nblocks, zero_init=False, out=out)
        assert torch.equal(out[1].cpu(), ecnt[lo:hi]), (d, R, K)
        assert bool(((out[0].cpu() - exp[lo:hi]).abs() <= tol[lo:hi]).all()), (d, R, K)
    with pytest.raises(RuntimeError):
        ops.voxel_bucket_exchange_cuda(pts[:10].to(DEV), feats[:10].to(DEV), kw["grid_min"], kw["voxel_size"], kw["grid_size"], R, K, 1,
                                       0, nblocks, *dest, ctas_per_sm=9)


@pytest.mark.gpu
@pytest.mark.parametrize("R", [1, 2, 3, 8])
@pytest.mark.parametrize("N", [0, 1, 5000, 60_000])
def test_sparse_reduce_with_every_rank_on_one_gpu(R, N, cuda_lib):
    """The sparse reduction's two calls with all ranks on this GPU: every source bins its shard into a private full
    grid (sums + counts), appends the occupied voxels of every other owner's slab to that owner's list, and every owner
    adds the lists to its own slab and normalises.  Each slab must equal the oracle's grid of the whole cloud.  The
    grid's voxel count is not a multiple of 4 or of the rank count, so ranges start at odd offsets."""
    kw = dict(grid_min=[-2.0, -2.0, -2.0], voxel_size=0.25, grid_size=[17, 15, 13])
    V = 17 * 15 * 13
    pts, feats = _cloud(N, 700 + R + N)
    cuts = [N * r // R for r in range(R + 1)]
    cap = V
    lists = [dict(ids=torch.full((R * cap,), -7, dtype=torch.int32, device=DEV), sums=torch.full((R * cap, 4), float("nan"), device=DEV),
                  cnts=torch.full((R * cap,), -1, dtype=torch.int32, device=DEV),
                  nrec=torch.full((R,), 12345, dtype=torch.int32, device=DEV)) for _ in range(R)]
    cursors = torch.zeros(16, dtype=torch.int32, device=DEV)
    overflow = torch.zeros(1, dtype=torch.int32, device=DEV)
    partial = []
    for r in range(R):
        g, c = ops.voxelize_pointcloud_cuda(pts[cuts[r]:cuts[r + 1]].to(DEV), feats[cuts[r]:cuts[r + 1]].to(DEV), kw["grid_min"],
                                            kw["voxel_size"], kw["grid_size"], "mean", normalize=False)
        g, c = g.view(V, 4), c.view(V)
        partial.append((g, c))
        others = [(r + k) % R for k in range(1, R)]
        ops.voxel_sparse_send_cuda(g, c, [sharding.slab_bounds(V, d, R) for d in others], cap,
                                   [lists[d]["ids"].data_ptr() + r * cap * 4 for d in others],
                                   [lists[d]["sums"].data_ptr() + r * cap * 16 for d in others],
                                   [lists[d]["cnts"].data_ptr() + r * cap * 4 for d in others],
                                   [lists[d]["nrec"].data_ptr() + r * 4 for d in others], cursors, overflow)
        assert int(overflow.item()) == 0
    if N:
        exp, ecnt, sabs = oracle.voxelize_pointcloud(pts, feats, mode="mean", return_aux=True, **kw)
        tol = oracle.mean_tolerance(ecnt, sabs, exp).reshape(V, 4)
        exp, ecnt = exp.reshape(V, 4), ecnt.reshape(V)
    else:
        exp, ecnt, tol = torch.zeros(V, 4), torch.zeros(V, dtype=torch.int32), torch.zeros(V, 4)
    for d in range(R):
        lo, hi = sharding.slab_bounds(V, d, R)
        srcs = [(d + k) % R for k in range(1, R)]
        g, c = partial[d]
        ops.voxel_sparse_merge_cuda([lists[d]["ids"].data_ptr() + s * cap * 4 for s in srcs],
                                    [lists[d]["sums"].data_ptr() + s * cap * 16 for s in srcs],
                                    [lists[d]["cnts"].data_ptr() + s * cap * 4 for s in srcs],
                                    [lists[d]["nrec"].data_ptr() + s * 4 for s in srcs], cap, g, c, lo, hi)
        assert torch.equal(c[lo:hi].cpu(), ecnt[lo:hi]), (d, R)
        assert bool(((g[lo:hi].cpu() - exp[lo:hi]).abs() <= tol[lo:hi]).all()), (d, R)
        # the number of records a source sent is the number of voxels it occupies in this slab
        for s_ in srcs:
            sent = int(lists[d]["nrec"][s_].item())
            # partial[s_] counts outside its own slab are untouched by any merge
            assert sent == int((partial[s_][1][lo:hi] > 0).sum()), (d, s_)


@pytest.mark.gpu
def test_sparse_reduce_overflow_is_reported_and_harmless(cuda_lib):
    """A record list that is too small: the published number still counts every occupied voxel, the overflow flag is
    raised, nothing is written past the list, and the merge reads no more than the capacity."""
    kw = dict(grid_min=[-2.0, -2.0, -2.0], voxel_size=0.25, grid_size=[16, 16, 16])
    V = 16 ** 3
    pts, feats = _cloud(20_000, 31)
    g, c = ops.voxelize_pointcloud_cuda(pts.to(DEV), feats.to(DEV), kw["grid_min"], kw["voxel_size"], kw["grid_size"], "mean",
                                        normalize=False)
    g, c = g.view(V, 4), c.view(V)
    cap = 100
    ids = torch.full((cap + 64,), -7, dtype=torch.int32, device=DEV)
    sums = torch.zeros(cap + 64, 4, device=DEV)
    cnts = torch.full((cap + 64,), -1, dtype=torch.int32, device=DEV)
    nrec = torch.zeros(1, dtype=torch.int32, device=DEV)
    cursors = torch.zeros(16, dtype=torch.int32, device=DEV)
    overflow = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.voxel_sparse_send_cuda(g, c, [(0, V)], cap, [ids.data_ptr()], [sums.data_ptr()], [cnts.data_ptr()], [nrec.data_ptr()],
                               cursors, overflow)
    occupied = int((c > 0).sum())
    assert occupied > cap and int(nrec.item()) == occupied and int(overflow.item()) == 1
    assert bool((ids[cap:] == -7).all()) and bool((cnts[cap:] == -1).all())
    assert bool((ids[:cap] >= 0).all())
    g2, c2 = torch.zeros(V, 4, device=DEV), torch.zeros(V, dtype=torch.int32, device=DEV)
    ops.voxel_sparse_merge_cuda([ids.data_ptr()], [sums.data_ptr()], [cnts.data_ptr()], [nrec.data_ptr()], cap, g2, c2, 0, V,
                                normalize=False)
    assert int((c2 > 0).sum()) == cap and int(c2.sum()) == int(cnts[:cap].sum())


@pytest.mark.gpu
@pytest.mark.parametrize("R", [2, 5])
def test_sparse_reduce_count_mode_on_one_gpu(R, cuda_lib):
    """Count mode of the sparse reduction: private count grids, (voxel id, count) records, no feature sums anywhere."""
    kw = dict(grid_min=[-2.0, -2.0, -2.0], voxel_size=0.25, grid_size=[17, 15, 13])
    V = 17 * 15 * 13
    N = 40_000
    pts, _ = _cloud(N, 77 + R)
    cuts = [N * r // R for r in range(R + 1)]
    cap = V
    lists = [dict(ids=torch.full((R * cap,), -7, dtype=torch.int32, device=DEV), cnts=torch.full((R * cap,), -1, dtype=torch.int32, device=DEV),
                  nrec=torch.zeros(R, dtype=torch.int32, device=DEV)) for _ in range(R)]
    cursors = torch.zeros(16, dtype=torch.int32, device=DEV)
    overflow = torch.zeros(1, dtype=torch.int32, device=DEV)
    partial = []
    for r in range(R):
        c = ops.voxelize_pointcloud_cuda(pts[cuts[r]:cuts[r + 1]].to(DEV), None, kw["grid_min"], kw["voxel_size"], kw["grid_size"],
                                         "count")[0].view(V)
        partial.append(c)
        others = [(r + k) % R for k in range(1, R)]
        ops.voxel_sparse_send_cuda(None, c, [sharding.slab_bounds(V, d, R) for d in others], cap,
                                   [lists[d]["ids"].data_ptr() + r * cap * 4 for d in others], [None] * len(others),
                                   [lists[d]["cnts"].data_ptr() + r * cap * 4 for d in others],
                                   [lists[d]["nrec"].data_ptr() + r * 4 for d in others], cursors, overflow)
    want = oracle.voxelize_pointcloud(pts, None, mode="count", **kw).reshape(V)
    for d in range(R):
        lo, hi = sharding.slab_bounds(V, d, R)
        srcs = [(d + k) % R for k in range(1, R)]
        ops.voxel_sparse_merge_cuda([lists[d]["ids"].data_ptr() + s * cap * 4 for s in srcs], [None] * len(srcs),
                                    [lists[d]["cnts"].data_ptr() + s * cap * 4 for s in srcs],
                                    [lists[d]["nrec"].data_ptr() + s * 4 for s in srcs], cap, None, partial[d], lo, hi)
        assert torch.equal(partial[d][lo:hi].cpu(), want[lo:hi]), (d, R)
    assert int(overflow.item()) == 0


@pytest.mark.gpu
def test_peer_barrier_passes_alone_and_gives_up_on_a_rank_that_never_arrives(cuda_lib):
    """The flag barrier's kernel on one GPU.  A world of one passes at once, epoch after epoch.  In a "world of two"
    whose second rank does not exist (its flag array is a buffer nobody writes) the wait runs out after the given number
    of polls, the kernel returns, the status word is raised and the context stays usable - the bounded wait that keeps
    a missing rank from hanging the others."""
    import ctypes
    VP1, VP2 = ctypes.c_void_p * 1, ctypes.c_void_p * 2
    flags = torch.zeros(32, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    stream = torch.cuda.current_stream().cuda_stream
    dev = torch.cuda.current_device()
    for epoch in (1, 2, 3):
        assert cuda_lib.rc_peer_barrier(VP1(flags.data_ptr()), 1, 0, epoch, status.data_ptr(), 0, dev, stream) == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and int(flags[0].item()) == 3
    absent = torch.zeros(32, dtype=torch.int32, device=DEV)        # "rank 1": never signals
    assert cuda_lib.rc_peer_barrier(VP2(flags.data_ptr(), absent.data_ptr()), 2, 0, 4, status.data_ptr(), 2000, dev, stream) == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 1                                 # gave up, reported it
    assert int(absent[0].item()) == 4                              # its own arrival did reach the other array
    x = torch.arange(10, device=DEV).sum().item()                  # the context is still usable
    assert x == 45
    # argument errors are reported before any launch
    assert cuda_lib.rc_peer_barrier(VP1(flags.data_ptr()), 1, 1, 1, None, 0, dev, stream) != 0
    assert cuda_lib.rc_peer_barrier(VP1(None), 1, 0, 1, None, 0, dev, stream) != 0
    assert cuda_lib.rc_peer_barrier(None, 1, 0, 1, None, 0, dev, stream) != 0
