"""rc_voxelize_mean_static: mean-mode voxelisation for callers that may not allocate device memory
(allocator callbacks, control loops that forbid driver allocations once running, hosts that own
only the buffers they were handed).  Its per-voxel counters sit in a fixed array inside the library
instead of a caller buffer.

The file is named to be collected last, so a run that stops at the first failure has already run
every other test.  It checks, through the C ABI, that two calls in a row (different clouds, so
stale counters from the first call would corrupt the second) agree with the ordinary entry point
and with the CPU oracle within the tolerance the other mean-mode tests use, that the largest grid
the fixed array covers (128^3) and a feature width that is not a multiple of four work, and that a
grid beyond the fixed capacity is refused.
"""
import ctypes

import pytest
import torch

import oracle
from robogoat_b200 import _lib

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _ordinary(L, pts, feats, gmin, vs, gs, F, flags=_lib.VOXEL_ZERO_INIT):
    V = gs[0] * gs[1] * gs[2]
    grid = torch.empty(V * F, dtype=torch.float32, device=DEV)
    counts = torch.empty(V, dtype=torch.int32, device=DEV)
    rc = L.rc_voxelize(pts.data_ptr(), feats.data_ptr(), grid.data_ptr(), counts.data_ptr(), pts.shape[0], F,
                       (ctypes.c_float * 3)(*gmin), vs, (ctypes.c_int32 * 3)(*gs), _lib.VOXEL_MEAN, flags, 0,
                       torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    return grid, counts


def _static(L, pts, feats, gmin, vs, gs, F):
    V = gs[0] * gs[1] * gs[2]
    grid = torch.full((V * F,), float("nan"), dtype=torch.float32, device=DEV)   # the call must clear it
    rc = L.rc_voxelize_mean_static(pts.data_ptr(), feats.data_ptr(), grid.data_ptr(), pts.shape[0], F,
                                   (ctypes.c_float * 3)(*gmin), vs, (ctypes.c_int32 * 3)(*gs), 0,
                                   torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    return grid


def test_static_counters_match_ordinary_entry_point_twice(cuda_lib):
    L = cuda_lib
    F = 4
    gmin, vs, gs = [-2.0, -2.0, -2.0], 0.125, [32, 32, 32]
    for call, (seed, n, scale) in enumerate([(11, 60_000, 4.0), (12, 35_000, 3.0)]):
        g = torch.Generator().manual_seed(seed)
        pts = (torch.rand(n, 3, generator=g) * scale - scale / 2).to(DEV)
        feats = torch.randn(n, F, generator=g).to(DEV)
        want, counts = _ordinary(L, pts, feats, gmin, vs, gs, F)
        # tolerance of the other mean tests: 1e-5 relative + 1e-6 * mean |feature| of the voxel
        abs_sums, _ = _ordinary(L, pts, feats.abs(), gmin, vs, gs, F, _lib.VOXEL_ZERO_INIT | _lib.VOXEL_NO_NORMALIZE)
        got = _static(L, pts, feats, gmin, vs, gs, F)
        torch.cuda.synchronize()
        c = counts.clamp(min=1).float().repeat_interleave(F)
        tol = 1e-5 * want.abs() + 1e-6 * abs_sums / c
        err = (got - want).abs()
        assert not torch.isnan(got).any(), f"call {call}: grid not cleared"
        assert bool((err <= tol).all()), f"call {call}: max excess {(err - tol).max().item()}"
        assert bool((got[(counts == 0).repeat_interleave(F)] == 0).all()), f"call {call}: empty voxels must be 0"
        # and against the CPU oracle, with the oracle's own tolerance
        em, ec, sabs = oracle.voxelize_pointcloud(pts.cpu(), feats.cpu(), gmin, vs, gs, mode="mean", return_aux=True)
        assert bool(((got.cpu().reshape(-1, F) - em.reshape(-1, F)).abs() <= oracle.mean_tolerance(ec, sabs, em).reshape(-1, F)).all()), call


@pytest.mark.parametrize("gs,F", [([128, 128, 128], 4), ([40, 24, 56], 3), ([16, 16, 16], 5)])
def test_capacity_edge_and_odd_feature_widths(gs, F, cuda_lib):
    """128^3 is exactly the fixed array's size and must be accepted; feature widths off the 16-byte path too.
    Two calls in a row again, each against the ordinary entry point and the oracle."""
    L = cuda_lib
    ext = max(gs) * 0.05
    gmin, vs = [-ext / 2] * 3, 0.05
    for seed in (21, 22):
        g = torch.Generator().manual_seed(seed + F)
        pts_h = torch.rand(50_000, 3, generator=g) * ext * 1.2 - ext * 0.6
        feats_h = torch.randn(50_000, F, generator=g)
        pts, feats = pts_h.to(DEV), feats_h.to(DEV)
        want, counts = _ordinary(L, pts, feats, gmin, vs, gs, F)
        got = _static(L, pts, feats, gmin, vs, gs, F)
        torch.cuda.synchronize()
        em, ec, sabs = oracle.voxelize_pointcloud(pts_h, feats_h, gmin, vs, gs, mode="mean", return_aux=True)
        tol = oracle.mean_tolerance(ec, sabs, em).reshape(-1, F)
        assert torch.equal(counts.cpu(), ec.reshape(-1))
        assert bool(((got.cpu().reshape(-1, F) - em.reshape(-1, F)).abs() <= tol).all()), seed
        assert bool(((got.cpu().reshape(-1, F) - want.cpu().reshape(-1, F)).abs() <= 2 * tol).all()), seed


def test_capacity_is_enforced(cuda_lib):
    L = cuda_lib
    pts = torch.zeros(4, 3, device=DEV)
    feats = torch.zeros(4, 4, device=DEV)
    grid = torch.zeros(16, device=DEV)
    too_big = (ctypes.c_int32 * 3)(129, 128, 128)          # one plane more than RC_STATIC_MAX_VOXELS
    rc = L.rc_voxelize_mean_static(pts.data_ptr(), feats.data_ptr(), grid.data_ptr(), 4, 4, (ctypes.c_float * 3)(0, 0, 0),
                                   0.1, too_big, 0, None)
    assert rc == 7 and b"exceeds" in L.rc_strerror(rc)
    assert _lib.STATIC_MAX_VOXELS == 128 ** 3
