"""Host logic of the multi-GPU harness on CPU: shard arithmetic, and the gather / reduce helpers run as
two gloo ranks.  The per-rank partial results are made with the CPU oracle here (in the product they
come from the CUDA kernels); what is under test is the partition rule and the collective semantics:
occupancy MAX, count SUM (exact), feature-sum SUM then normalise, batch-row gather."""
import datetime
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from robogoat_b200 import sharding
import workloads


def test_shard_bounds_partition():
    for n in (0, 1, 7, 4096, 16385):
        for ws in (1, 2, 3, 4, 8):
            spans = [sharding.shard_bounds(n, r, ws) for r in range(ws)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            for (a, b), (c, d) in zip(spans, spans[1:]):
                assert b == c and a <= b
            per = (n + ws - 1) // ws
            assert all(b - a <= per for a, b in spans)
    assert sharding.shard_bounds(4096, 7, 8) == (3584, 4096)
    assert sharding.shard_bounds(16384, 3, 8) == (6144, 8192)
    with pytest.raises(ValueError):
        sharding.shard_bounds(10, 2, 2)
    assert sharding.world() == (0, 1)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, ws, port, fn, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=ws, timeout=datetime.timedelta(seconds=60))
    try:
        ret[rank] = fn(rank, ws)
    finally:
        dist.destroy_process_group()


def _run(fn, ws=2):
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, ws, port, fn, ret)) for r in range(ws)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    return dict(ret)


def _batch_job(rank, ws):
    B = 7                                                       # odd: the last shard is shorter
    src, st, tt = workloads.resample_inputs(B=B, S=40, D=12, T=9, irregular_targets=True, seed=3)
    full = oracle.resample_trajectories(src, st, tt)
    s, t, q = sharding.shard_rows([src, st, tt], rank, ws)
    local = oracle.resample_trajectories(s, t, q) if s.shape[0] else torch.empty(0, 9, 12)
    got = sharding.gather_rows(local, B)
    return bool(torch.equal(got, full)) and local.shape[0] == (4 if rank == 0 else 3)


def _voxel_job(rank, ws):
    g = torch.Generator().manual_seed(9)
    pts = torch.rand(20_001, 3, generator=g) * 4 - 2
    feats = torch.randn(20_001, 4, generator=g)
    kw = dict(grid_min=[-1.5, -1.5, -1.5], voxel_size=0.25, grid_size=[12, 12, 12])
    a, b = sharding.shard_bounds(pts.shape[0], rank, ws)
    ok = True
    for mode in ("occupancy", "count"):
        full = oracle.voxelize_pointcloud(pts, None, mode=mode, **kw)
        part = oracle.voxelize_pointcloud(pts[a:b], None, mode=mode, **kw)
        sharding.reduce_partial_grids(part, None, mode)
        ok = ok and bool(torch.equal(part, full))
    full, fcnt, sabs = oracle.voxelize_pointcloud(pts, feats, mode="mean", return_aux=True, **kw)
    mean, cnt, _ = oracle.voxelize_pointcloud(pts[a:b], feats[a:b], mode="mean", return_aux=True, **kw)
    sums = mean * cnt.unsqueeze(-1)                             # partial feature sums of this rank
    sharding.reduce_partial_grids(sums, cnt, "mean")
    ok = ok and bool(torch.equal(cnt, fcnt))
    merged = torch.where(cnt.unsqueeze(-1) > 0, sums * (1.0 / cnt.clamp(min=1)).unsqueeze(-1), torch.zeros_like(sums))
    tol = oracle.mean_tolerance(fcnt, sabs, full) + 1e-6
    ok = ok and bool(((merged - full).abs() <= tol).all())
    try:
        sharding.reduce_partial_grids(sums, None, "mean")
        ok = False
    except RuntimeError:
        pass
    return ok


def _max_job(rank, ws):
    """Max mode with all-negative features and spatially disjoint shards: a rank's decoded max grid holds 0.0
    where it saw no point, and that 0.0 must not beat the other rank's negative maximum."""
    g = torch.Generator().manual_seed(17)
    pts = torch.rand(4_000, 3, generator=g) * 3 - 1.5
    pts[:, 2] = torch.where(torch.arange(4_000) < 2_000, pts[:, 2].abs() * -1 - 0.01, pts[:, 2].abs() + 0.01)  # rank 0 below z=0, rank 1 above
    feats = -torch.rand(4_000, 3, generator=g) - 0.5                                                          # all negative
    kw = dict(grid_min=[-1.5, -1.5, -1.5], voxel_size=0.25, grid_size=[12, 12, 12])
    V = 12 ** 3

    def decoded_max(p, f):     # what the single-GPU operator returns: true maximum, empty voxels 0.0
        ids = oracle.voxel_ids(p, **kw)
        keep = ids >= 0
        out = torch.full((V, 3), float("-inf")).scatter_reduce_(0, ids[keep].long().unsqueeze(1).expand(-1, 3), f[keep], "amax")
        occ = torch.zeros(V, dtype=torch.uint8)
        occ[ids[keep].long()] = 1
        return torch.where(occ.bool().unsqueeze(1), out, torch.zeros_like(out)), occ

    full, _ = decoded_max(pts, feats)
    a, b = sharding.shard_bounds(4_000, rank, ws)
    part, occ = decoded_max(pts[a:b], feats[a:b])
    naive = part.clone()
    sharding.reduce_partial_grids(naive, None, "max")          # without the masks: the 0.0 of an empty voxel wins
    sharding.mask_empty_for_max(part, occ)
    sharding.reduce_partial_grids(part, None, "max")
    sharding.reduce_partial_grids(occ, None, "occupancy")
    sharding.unmask_empty_after_max(part, occ)
    return bool(torch.equal(part, full)) and not bool(torch.equal(naive, full)) and bool((full < 0).any())


def test_sharded_max_keeps_negative_maxima():
    assert _run(_max_job) == {0: True, 1: True}


def test_batch_shards_gather_to_the_unsharded_result():
    assert _run(_batch_job) == {0: True, 1: True}


def test_partial_grids_reduce_to_the_single_process_grid():
    assert _run(_voxel_job) == {0: True, 1: True}


def _exchange_job(rank, ws):
    """Point exchange on CPU: the oracle's voxel ids bucketed with a stable sort stand in for the partition
    kernel; what is checked is the all-to-all bookkeeping and that the owner's slab comes out right."""
    g = torch.Generator().manual_seed(21)
    pts = torch.rand(9_001, 3, generator=g) * 4 - 2
    feats = torch.randn(9_001, 4, generator=g)
    kw = dict(grid_min=[-1.5, -1.5, -1.5], voxel_size=0.25, grid_size=[12, 12, 11])    # V = 1584, slabs of 792
    V = 12 * 12 * 11
    a, b = sharding.shard_bounds(pts.shape[0], rank, ws)
    ids = oracle.voxel_ids(pts[a:b], **kw)
    keep = ids >= 0
    ids_k, f_k = ids[keep].to(torch.int32), feats[a:b][keep]
    per = (V + ws - 1) // ws
    owner = ids_k.long() // per
    order = torch.sort(owner, stable=True).indices
    send = torch.bincount(owner, minlength=ws).tolist()
    (ids_in, f_in), recv = sharding.exchange_buckets([ids_k[order], f_k[order]], send)
    lo, hi = sharding.slab_bounds(V, rank, ws)
    ok = len(recv) == ws and ids_in.shape[0] == sum(recv) and bool(((ids_in >= lo) & (ids_in < hi)).all())
    cnt = torch.bincount((ids_in - lo).long(), minlength=hi - lo)
    full = oracle.voxelize_pointcloud(pts, None, mode="count", **kw).reshape(-1)
    ok = ok and bool(torch.equal(cnt.int(), full[lo:hi]))
    sums = torch.zeros(hi - lo, 4, dtype=torch.float64).index_add_(0, (ids_in - lo).long(), f_in.double())
    all_ids = oracle.voxel_ids(pts, **kw)
    exp_sums = torch.zeros(V, 4, dtype=torch.float64).index_add_(0, all_ids[all_ids >= 0].long(), feats[all_ids >= 0].double())
    ok = ok and bool(torch.allclose(sums, exp_sums[lo:hi], rtol=1e-12, atol=1e-12))
    try:
        sharding.exchange_buckets([ids_k], send[:-1])
        ok = False
    except RuntimeError:
        pass
    return ok


def test_point_exchange_delivers_every_point_to_the_owner_of_its_voxel():
    assert _run(_exchange_job) == {0: True, 1: True}
    assert sharding.slab_bounds(1584, 1, 2) == (792, 1584)
    one, counts = sharding.exchange_buckets([torch.arange(10)], [7])        # no process group: identity on the prefix
    assert torch.equal(one[0], torch.arange(7)) and counts == [7]


def test_exchange_plan_bookkeeping():
    """Count matrix -> send/receive sizes, the layout of the receive buffer and every sender's first slot in it."""
    R, K = 3, 2
    g = torch.Generator().manual_seed(4)
    C = torch.randint(0, 50, (R, R * K), generator=g).tolist()
    plans = [sharding.exchange_plan(C, r, K) for r in range(R)]
    for d in range(R):
        assert plans[d]["recv_counts"] == [plans[s]["send_counts"][d] for s in range(R)]
        assert sum(c for _, c, _ in plans[d]["runs"]) == plans[d]["totals"][d] == sum(plans[d]["recv_counts"])
        # replay the writes of every sender into owner d's buffer: every slot is hit exactly once, by the run the owner expects
        slots = [None] * plans[d]["totals"][d]
        for s in range(R):
            for k in range(K):
                first = plans[s]["dest_start"][d * K + k]
                for j in range(C[s][d * K + k]):
                    assert slots[first + j] is None
                    slots[first + j] = (s, k)
        assert all(x is not None for x in slots)
        for (off, cnt, k), (s, kk) in zip(plans[d]["runs"], [(s, k) for s in range(R) for k in range(K)]):
            assert k == kk and all(slots[off + j] == (s, k) for j in range(cnt))
    assert all(p["totals"] == plans[0]["totals"] for p in plans)
    assert sharding.sub_parts(512 ** 3, 4, 8, "mean") == 4 and sharding.sub_parts(512 ** 3, 4, 2, "mean") == 14
    assert sharding.sub_parts(128 ** 3, 0, 2, "count") == 1 and sharding.sub_parts(512 ** 3, 0, 64, "count") == 1
    assert sharding.sub_parts(10 ** 9, 16, 2, "mean") == 32 and sharding.sub_parts(512 ** 3, 4, 8, "occupancy") == 1


def test_batched_exchange_plans_lay_the_batches_out_back_to_back():
    """Batched direct exchange: per batch the plan of that batch, shifted behind the records of the batches before
    it in every owner's buffer; replaying all stores hits every slot once, and the owner's runs name the right slots."""
    R, K, nb = 3, 2, 4
    g = torch.Generator().manual_seed(6)
    C = torch.randint(0, 40, (R, nb, R * K), generator=g).tolist()          # [source][batch][part]
    per_rank = [sharding.batched_exchange_plans(C, r, K) for r in range(R)]
    assert all(t == per_rank[0][1] for _, t in per_rank)
    totals = per_rank[0][1]
    for d in range(R):
        slots = [None] * totals[d]
        for s in range(R):
            for i in range(nb):
                starts = per_rank[s][0][i]["dest_start"]
                for k in range(K):
                    for j in range(C[s][i][d * K + k]):
                        assert slots[starts[d * K + k] + j] is None
                        slots[starts[d * K + k] + j] = (i, s, k)
        assert all(x is not None for x in slots)
        for i in range(nb):
            for (off, cnt, k), (s, kk) in zip(per_rank[d][0][i]["runs"], [(s, k) for s in range(R) for k in range(K)]):
                assert k == kk and all(slots[off + j] == (i, s, k) for j in range(cnt))


def _lonely_rank(port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    try:
        dist.init_process_group("gloo", rank=0, world_size=2, timeout=datetime.timedelta(seconds=3))
        t = torch.ones(4)
        dist.all_reduce(t)
        q.put("completed")
    except Exception as e:  # the missing peer must surface as an error on the host, not a hang
        q.put("error:" + type(e).__name__)


def test_a_rank_that_never_joins_is_reported_not_waited_for_forever():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    p = ctx.Process(target=_lonely_rank, args=(_free_port(), q))
    p.start()
    p.join(60)
    assert not p.is_alive(), "rendezvous did not time out"
    assert q.get(timeout=5).startswith("error:")


def test_bucket_slice_windows_tile_every_ranks_blocks_exactly():
    """The sliced bucket exchange's bookkeeping: over all slices the windows of a source rank cover its blocks of the
    owner's pool once, in order, without reaching into the next rank's; points map to chunks 1024 at a time."""
    for chunks, ranks, slices in [(0, 2, 3), (1, 2, 4), (7, 3, 3), (64, 8, 4), (65, 4, 8), (100, 2, 16), (5, 16, 1)]:
        covered = {r: [] for r in range(ranks)}
        chunk_runs = []
        for s in range(slices):
            first, n, blocks = sharding.bucket_slice_windows(chunks, ranks, slices, s)
            assert 0 <= first <= chunks and 0 <= n and first + n <= chunks
            assert blocks == [r * chunks + first for r in range(ranks)]
            chunk_runs.append((first, n))
            for r in range(ranks):
                covered[r] += list(range(blocks[r], blocks[r] + n))
        for r in range(ranks):
            assert covered[r] == list(range(r * chunks, (r + 1) * chunks)), (chunks, ranks, slices, r)
        assert sum(n for _, n in chunk_runs) == chunks
        sizes = [n for _, n in chunk_runs]
        assert sizes == sorted(sizes, reverse=True)                     # full runs first, one short run, then empty slices
        assert len({n for n in sizes if n and n != sizes[0]}) <= 1
    import pytest
    with pytest.raises(ValueError):
        sharding.bucket_slice_windows(8, 2, 4, 4)
    with pytest.raises(ValueError):
        sharding.bucket_slice_windows(8, 0, 4, 0)


def test_sparse_list_offsets_pair_every_writer_with_one_reader():
    """The sparse reduction's bookkeeping: rank a writes its list for owner b where b reads the list of source a; the
    lists inside a pool do not overlap; everybody starts with its neighbour."""
    for ranks in (1, 2, 3, 8, 16):
        cap = 1000
        views = [sharding.sparse_list_offsets(r, ranks, cap) for r in range(ranks)]
        for a in range(ranks):
            others, write_at, read_at = views[a]
            assert sorted(others) == [r for r in range(ranks) if r != a]
            assert not others or others[0] == (a + 1) % ranks
            assert write_at == a * cap and len(set(read_at)) == len(read_at)
            for b, off in zip(others, read_at):
                assert off == views[b][1]                      # where a reads b's list is where b wrote it
                assert off % cap == 0 and off // cap == b
    import pytest
    with pytest.raises(ValueError):
        sharding.sparse_list_offsets(2, 2, 10)


def test_auto_form_falls_back_only_on_overflow(monkeypatch):
    """Host logic of ``voxelize_sharded_auto`` with the two GPU forms replaced by stand-ins: a record-list overflow sends
    the call to the bucket exchange, any other error - and an overflow report that comes with a barrier time-out -
    reaches the caller."""
    class Lists:
        barrier = None
        last_form = None

    class TimedOut:
        def timed_out(self):
            return True

    calls = []

    def sparse_ok(*a, **k):
        calls.append("sparse")
        return "S"

    def sparse_overflow(*a, **k):
        calls.append("sparse")
        raise RuntimeError("sparse reduction: a record list of 8 records overflowed on some rank, or a barrier gave up")

    def sparse_broken(*a, **k):
        raise RuntimeError("voxel_sparse_send: invalid device pointer")

    def buckets(*a, **k):
        calls.append("buckets")
        return "B"

    monkeypatch.setattr(sharding, "voxelize_sharded_buckets", buckets)
    lists = Lists()
    monkeypatch.setattr(sharding, "voxelize_sharded_sparse", sparse_ok)
    assert sharding.voxelize_sharded_auto(None, None, lists, None) == "S" and lists.last_form == "sparse"
    monkeypatch.setattr(sharding, "voxelize_sharded_sparse", sparse_overflow)
    assert sharding.voxelize_sharded_auto(None, None, lists, None) == "B" and lists.last_form == "buckets"
    assert calls == ["sparse", "sparse", "buckets"]
    monkeypatch.setattr(sharding, "voxelize_sharded_sparse", sparse_broken)
    with pytest.raises(RuntimeError, match="invalid device pointer"):
        sharding.voxelize_sharded_auto(None, None, lists, None)
    lists.barrier = TimedOut()
    monkeypatch.setattr(sharding, "voxelize_sharded_sparse", sparse_overflow)
    with pytest.raises(RuntimeError, match="overflowed"):
        sharding.voxelize_sharded_auto(None, None, lists, None)
