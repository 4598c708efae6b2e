"""Sharded operators on real GPUs (needs at least two): launched as child processes over NCCL, results
compared with a single-GPU run of the same inputs.  NVLS is switched off for these short-lived children."""
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["REPO_ROOT"])
from robogoat_b200 import sharding, workloads, ops
import robocache
rank, ws = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
dev = torch.device("cuda", rank)
src, st, tt = workloads.resample_inputs(B=37, S=100, D=64, T=50, dtype=torch.bfloat16, irregular_targets=True, seed=1)
full = robocache.resample_trajectories(src.to(dev), st.to(dev), tt.to(dev))
got = sharding.resample_sharded(src, st, tt, gather=True)
assert torch.equal(got.view(torch.int16), full.view(torch.int16)), "resample"
a = workloads.fusion_inputs(B=19, dtype=torch.bfloat16, seed=2)
full = robocache.fuse_multimodal(*[x.to(dev) for x in a])
got = sharding.fuse_sharded(*a, gather=True)
assert torch.equal(got.view(torch.int16), full.view(torch.int16)), "fusion"
g = torch.Generator().manual_seed(3)
pts = (torch.rand(200_003, 3, generator=g) * 4 - 2).to(dev)
feats = torch.randn(200_003, 4, generator=g).to(dev)
kw = dict(grid_min=[-1.5, -1.5, -1.5], voxel_size=0.125, grid_size=[24, 24, 24])
lo, hi = sharding.shard_bounds(pts.shape[0], rank, ws)
for mode in ("occupancy", "count"):
    full = robocache.voxelize_pointcloud(pts, mode=mode, **kw)
    got = sharding.voxelize_sharded(pts[lo:hi], None, mode=mode, **kw)
    assert got.dtype == torch.int32 and torch.equal(got, full), mode
full, cnt = ops.voxelize_pointcloud_cuda(pts, feats, kw["grid_min"], kw["voxel_size"], kw["grid_size"], "mean")
sabs, _ = ops.voxelize_pointcloud_cuda(pts, feats.abs(), kw["grid_min"], kw["voxel_size"], kw["grid_size"], "mean", normalize=False)
tol = 1e-5 * full.abs() + 1e-6 * sabs / cnt.clamp(min=1).unsqueeze(-1)
for slab in (False, True):
    got = sharding.voxelize_sharded(pts[lo:hi], feats[lo:hi], mode="mean", slab_normalize=slab, **kw)
    assert bool(((got - full).abs() <= tol).all()), f"mean slab={slab}"
V = 24 ** 3
for mode in ("count", "mean"):
    slab = sharding.voxelize_sharded_slab(pts[lo:hi], feats[lo:hi] if mode == "mean" else None, mode=mode, **kw)
    a, b = rank * V // ws, (rank + 1) * V // ws
    if mode == "count":
        assert torch.equal(slab, robocache.voxelize_pointcloud(pts, mode="count", **kw).reshape(V)[a:b]), "slab count"
    else:
        assert bool(((slab - full.reshape(V, 4)[a:b]).abs() <= tol.reshape(V, 4)[a:b]).all()), "slab mean"
for mode in ("occupancy", "count", "mean"):                       # point exchange: the owner's slab, no dense grid
    slab = sharding.voxelize_sharded_exchange(pts[lo:hi], feats[lo:hi] if mode == "mean" else None, mode=mode, **kw)
    a, b = sharding.slab_bounds(V, rank, ws)
    if mode == "mean":
        assert bool(((slab - full.reshape(V, 4)[a:b]).abs() <= tol.reshape(V, 4)[a:b]).all()), "exchange mean"
    else:
        assert torch.equal(slab, robocache.voxelize_pointcloud(pts, mode=mode, **kw).reshape(V)[a:b]), "exchange " + mode
# direct form: the partition kernel stores into the owners' receive buffers (peer memory) itself; twice in a row, so
# that the second call's stores meet buffers the owners have just read, then with a buffer that is too small (falls back)
px = sharding.PointExchange(capacity=pts.shape[0], feature_width=4)
for rep in range(2):
    for mode in ("occupancy", "count", "mean"):
        slab = sharding.voxelize_sharded_exchange(pts[lo:hi], feats[lo:hi] if mode == "mean" else None, mode=mode, direct=px, **kw)
        a, b = sharding.slab_bounds(V, rank, ws)
        if mode == "mean":
            assert bool(((slab - full.reshape(V, 4)[a:b]).abs() <= tol.reshape(V, 4)[a:b]).all()), "direct mean"
        else:
            assert torch.equal(slab, robocache.voxelize_pointcloud(pts, mode=mode, **kw).reshape(V)[a:b]), "direct " + mode
px.close()
small = sharding.PointExchange(capacity=10, feature_width=4)
slab = sharding.voxelize_sharded_exchange(pts[lo:hi], None, mode="count", direct=small, **kw)
a, b = sharding.slab_bounds(V, rank, ws)
assert torch.equal(slab, robocache.voxelize_pointcloud(pts, mode="count", **kw).reshape(V)[a:b]), "fallback"
small.close()
torch.cuda.synchronize()
dist.barrier()
dist.destroy_process_group()
print("child ok", rank)
'''


def test_sharded_operators_match_single_gpu(cuda_lib):
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
    outs = [p.communicate(timeout=300)[0].decode() for p in procs]
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and f"child ok {r}" in o, o[-2000:]
