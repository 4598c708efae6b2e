"""Re-entrancy: the operators are called from several host threads, each on its own CUDA stream, as the
reference's stress test does (robocache/tests/stress/test_concurrent.py:12-70); every thread must get the
bits a single-threaded call produces."""
import threading

import pytest
import torch

import robocache
import workloads

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_four_threads_four_streams(cuda_lib):
    src, st, tt = (x.to(DEV) for x in workloads.resample_inputs(B=64, S=200, D=128, T=100, dtype=torch.bfloat16,
                                                                 irregular_targets=True, seed=8))
    fa = [x.to(DEV) for x in workloads.fusion_inputs(B=32, dtype=torch.bfloat16, seed=9)]
    pts = workloads.voxel_uniform_inputs(200_000, seed=10).to(DEV)
    kw = dict(grid_min=[-10.0, -10.0, -10.0], voxel_size=0.25, grid_size=[80, 80, 80])
    want = (robocache.resample_trajectories(src, st, tt), robocache.fuse_multimodal(*fa),
            robocache.voxelize_pointcloud(pts, mode="count", **kw))
    torch.cuda.synchronize()
    errors = []

    def worker(i):
        try:
            stream = torch.cuda.Stream(DEV)
            with torch.cuda.stream(stream):
                for _ in range(25):
                    r = robocache.resample_trajectories(src, st, tt)
                    f = robocache.fuse_multimodal(*fa)
                    v = robocache.voxelize_pointcloud(pts, mode="count", **kw)
                stream.synchronize()
                assert torch.equal(r.view(torch.int16), want[0].view(torch.int16))
                assert torch.equal(f.view(torch.int16), want[1].view(torch.int16))
                assert torch.equal(v, want[2])
        except Exception as e:  # surfaced in the main thread below
            errors.append((i, repr(e)))

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(4)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
