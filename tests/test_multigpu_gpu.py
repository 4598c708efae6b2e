"""Sharded operators on real GPUs (needs at least two): launched as child processes over NCCL, every result
compared with the CPU oracle run on the unsharded inputs (bit-exact for resampling, fusion, occupancy and counts;
means within the oracle's tolerance).  NVLS is switched off for these short-lived children."""
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r'''
import datetime, os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["REPO_ROOT"])
import oracle
from robogoat_b200 import sharding, ops
import workloads
import robocache
rank, ws = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
# a short timeout: should the other rank fail an assertion and leave, this one aborts by itself
dist.init_process_group("nccl", device_id=torch.device("cuda", rank), timeout=datetime.timedelta(seconds=90))
dev = torch.device("cuda", rank)
src, st, tt = workloads.resample_inputs(B=37, S=100, D=64, T=50, dtype=torch.bfloat16, irregular_targets=True, seed=1)
exp = oracle.round_to_bf16(oracle.resample_trajectories(src, st, tt))
got = sharding.resample_sharded(src, st, tt, gather=True)
assert torch.equal(got.cpu().view(torch.int16), exp.view(torch.int16)), "resample"
a = workloads.fusion_inputs(B=19, dtype=torch.bfloat16, seed=2)
exp = oracle.round_to_bf16(oracle.fuse_multimodal(*a))
got = sharding.fuse_sharded(*a, gather=True)
assert torch.equal(got.cpu().view(torch.int16), exp.view(torch.int16)), "fusion"
g = torch.Generator().manual_seed(3)
pts_h = torch.rand(200_003, 3, generator=g) * 4 - 2
feats_h = torch.randn(200_003, 4, generator=g)
pts, feats = pts_h.to(dev), feats_h.to(dev)
kw = dict(grid_min=[-1.5, -1.5, -1.5], voxel_size=0.125, grid_size=[24, 24, 24])
V = 24 ** 3
lo, hi = sharding.shard_bounds(pts.shape[0], rank, ws)
want = {m: oracle.voxelize_pointcloud(pts_h, None, mode=m, **kw) for m in ("occupancy", "count")}
mean, cnt, sabs = oracle.voxelize_pointcloud(pts_h, feats_h, mode="mean", return_aux=True, **kw)
tol = oracle.mean_tolerance(cnt, sabs, mean)
def mean_ok(got, a=0, b=V):
    return bool(((got.cpu().reshape(-1, 4) - mean.reshape(V, 4)[a:b]).abs() <= tol.reshape(V, 4)[a:b]).all())
for mode in ("occupancy", "count"):
    got = sharding.voxelize_sharded(pts[lo:hi], None, mode=mode, **kw)
    assert got.dtype == torch.int32 and torch.equal(got.cpu(), want[mode]), mode
for slab in (False, True):
    got = sharding.voxelize_sharded(pts[lo:hi], feats[lo:hi], mode="mean", slab_normalize=slab, **kw)
    assert mean_ok(got), f"mean slab={slab}"
# max mode with negative features: a voxel seen by one rank only keeps its (negative) maximum
neg = -feats_h.abs() - 0.25
ids = oracle.voxel_ids(pts_h, **kw)
keep = ids >= 0
mx = torch.full((V, 4), float("-inf")).scatter_reduce_(0, ids[keep].long().unsqueeze(1).expand(-1, 4), neg[keep], "amax")
mx = torch.where(torch.isinf(mx), torch.zeros_like(mx), mx)
got = sharding.voxelize_sharded(pts[lo:hi], neg.to(dev)[lo:hi], mode="max", **kw)
assert torch.equal(got.cpu().reshape(V, 4), mx), "max"
got = sharding.voxelize_sharded_slab(pts[lo:hi], neg.to(dev)[lo:hi], mode="max", **kw)
assert torch.equal(got.cpu(), mx[rank * V // ws:(rank + 1) * V // ws]), "slab max"
for mode in ("count", "mean"):
    slab = sharding.voxelize_sharded_slab(pts[lo:hi], feats[lo:hi] if mode == "mean" else None, mode=mode, **kw)
    a, b = rank * V // ws, (rank + 1) * V // ws
    if mode == "count":
        assert torch.equal(slab.cpu(), want["count"].reshape(V)[a:b]), "slab count"
    else:
        assert mean_ok(slab, a, b), "slab mean"
for mode in ("occupancy", "count", "mean"):                       # point exchange: the owner's slab, no dense grid
    slab = sharding.voxelize_sharded_exchange(pts[lo:hi], feats[lo:hi] if mode == "mean" else None, mode=mode, **kw)
    a, b = sharding.slab_bounds(V, rank, ws)
    if mode == "mean":
        assert mean_ok(slab, a, b), "exchange mean"
    else:
        assert torch.equal(slab.cpu(), want[mode].reshape(V)[a:b]), "exchange " + mode
# direct form: the partition kernel stores into the owners' receive buffers (peer memory) itself; twice in a row, so
# that the second call's stores meet buffers the owners have just read, then with a buffer that is too small (falls back)
px = sharding.PointExchange(capacity=pts.shape[0], feature_width=4)
for rep in range(2):
    for mode in ("occupancy", "count", "mean"):
        slab = sharding.voxelize_sharded_exchange(pts[lo:hi], feats[lo:hi] if mode == "mean" else None, mode=mode, direct=px, **kw)
        a, b = sharding.slab_bounds(V, rank, ws)
        if mode == "mean":
            assert mean_ok(slab, a, b), "direct mean"
        else:
            assert torch.equal(slab.cpu(), want[mode].reshape(V)[a:b]), "direct " + mode
# the same in slices of the local cloud whose stores and accumulation overlap on two streams
for batches in (2, 3):
    for mode in ("count", "mean"):
        slab = sharding.voxelize_sharded_exchange(pts[lo:hi], feats[lo:hi] if mode == "mean" else None, mode=mode, direct=px,
                                                  batches=batches, **kw)
        a, b = sharding.slab_bounds(V, rank, ws)
        if mode == "mean":
            assert mean_ok(slab, a, b), f"batched direct mean {batches}"
        else:
            assert torch.equal(slab.cpu(), want[mode].reshape(V)[a:b]), f"batched direct count {batches}"
px.close()
# bucket form: fixed blocks in the owners' pools, no counts and no host synchronisation; three calls in a row with
# different clouds, so that a call's stores meet pools the owners have just read
spans = [sharding.shard_bounds(pts_h.shape[0], r, ws) for r in range(ws)]
for fetch in (True, False):                 # owners fetch the records over NVLink / sources store them over NVLink
    bx = sharding.BucketExchange(points_per_rank=120_000, n_voxels=V, fetch=fetch)
    for rep, frac in enumerate((1, 3, 1)):
        used = [(l, l + (h - l) // frac) for l, h in spans]                 # every rank passes the first 1/frac of its shard
        sub_h = torch.cat([pts_h[l:h] for l, h in used])
        sub_f = torch.cat([feats_h[l:h] for l, h in used])
        m2, c2, s2 = oracle.voxelize_pointcloud(sub_h, sub_f, mode="mean", return_aux=True, **kw)
        t2 = oracle.mean_tolerance(c2, s2, m2).reshape(V, 4)
        l, h = used[rank]
        a, b = sharding.slab_bounds(V, rank, ws)
        # in one piece, then in slices whose accumulation overlaps the next slice's stores (storing form)
        for slices in ((1,) if fetch else (1, 3, 8)):
            slab, cnts = sharding.voxelize_sharded_buckets(pts[l:h], feats[l:h], bx, return_counts=True, slices=slices, **kw)
            assert torch.equal(cnts.cpu(), c2.reshape(V)[a:b]), f"bucket counts {rep} fetch={fetch} slices={slices}"
            assert bool(((slab.cpu() - m2.reshape(V, 4)[a:b]).abs() <= t2[a:b]).all()), f"bucket mean {rep} fetch={fetch} slices={slices}"
    assert not bx.barrier_timed_out()
    bx.close()
# sparse reduction: private full grids, only occupied voxels travel; twice in a row, then with lists that are too small
for barrier in ("peer", "nccl"):             # the flag kernel over NVLink / a 4-byte all-reduce
  sr = sharding.SparseReduce(records_per_pair=V, barrier=barrier)
  for rep in range(2):
      l, h = spans[rank]
      slab, cnts = sharding.voxelize_sharded_sparse(pts[l:h], feats[l:h], sr, return_counts=True, **kw)
      a, b = sharding.slab_bounds(V, rank, ws)
      assert torch.equal(cnts.cpu(), cnt.reshape(V)[a:b]), f"sparse counts {rep}"
      assert mean_ok(slab, a, b), f"sparse mean {rep}"
      cslab = sharding.voxelize_sharded_sparse(pts[l:h], None, sr, mode="count", **kw)
      assert cslab.dtype == torch.int32 and torch.equal(cslab.cpu(), want["count"].reshape(V)[a:b]), f"sparse count {rep}"
  assert not (sr.barrier is not None and sr.barrier.timed_out()), barrier
  sr.close()
# replicated output (what the dense all-reduce returns) by a sparse all-gather: lists stay with their sources, every rank
# merges the others' lists over NVLink into its own full grid
sg = sharding.SparseGather(records_per_rank=V)
for rep in range(2):
    l, h = spans[rank]
    for mode in ("occupancy", "count"):
        got = sharding.voxelize_sharded_sparse_full(pts[l:h], None, sg, mode=mode, **kw)
        assert got.dtype == torch.int32 and torch.equal(got.cpu(), want[mode]), f"sparse all-gather {mode} {rep}"
    got = sharding.voxelize_sharded_sparse_full(pts[l:h], feats[l:h], sg, mode="mean", **kw)
    assert mean_ok(got), f"sparse all-gather mean {rep}"
assert not sg.barrier.timed_out()
sg.close()
tiny = sharding.SparseReduce(records_per_pair=8)
try:
    sharding.voxelize_sharded_sparse(pts[l:h], feats[l:h], tiny, **kw)
    raise AssertionError("overflow not reported")
except RuntimeError as e:
    assert "overflowed" in str(e), e
# the form that picks by trying: lists that hold the cloud -> sparse reduction; lists that do not -> bucket exchange
roomy = sharding.SparseReduce(records_per_pair=V)
abx = sharding.BucketExchange(points_per_rank=120_000, n_voxels=V)
a, b = sharding.slab_bounds(V, rank, ws)
for lists, form in ((roomy, "sparse"), (tiny, "buckets"), (roomy, "sparse")):
    slab, cnts = sharding.voxelize_sharded_auto(pts[l:h], feats[l:h], lists, abx, return_counts=True, **kw)
    assert lists.last_form == form, (lists.last_form, form)
    assert torch.equal(cnts.cpu(), cnt.reshape(V)[a:b]) and mean_ok(slab, a, b), f"auto form {form}"
abx.close()
roomy.close()
tiny.close()
small = sharding.PointExchange(capacity=10, feature_width=4)
slab = sharding.voxelize_sharded_exchange(pts[lo:hi], None, mode="count", direct=small, **kw)
a, b = sharding.slab_bounds(V, rank, ws)
assert torch.equal(slab.cpu(), want["count"].reshape(V)[a:b]), "fallback"
small.close()
torch.cuda.synchronize()
dist.barrier()
dist.destroy_process_group()
print("child ok", rank)
'''


def test_sharded_operators_match_the_oracle(cuda_lib):
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least two GPUs")
    ws = 2
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    procs = []
    for r in range(ws):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(ws), LOCAL_RANK=str(r), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), REPO_ROOT=ROOT, NCCL_NVLS_ENABLE="0")
        procs.append(subprocess.Popen([sys.executable, "-c", CHILD], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT))
    outs = []
    try:
        for p in procs:
            outs.append(p.communicate(timeout=300)[0].decode())
    finally:
        for p in procs:             # a child still running here is stuck behind a rank that has left: end it (NVLS is off)
            if p.poll() is None:
                p.kill()
                p.wait()
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and f"child ok {r}" in o, o[-2000:]
