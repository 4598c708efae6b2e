"""Checks the oracle's voxel binning against the reference's own C++ header
(robocache/validation/cpu_reference.hpp) compiled unmodified behind oracle/ref_shim.cpp.
Skipped where that library was not built (it needs a reference checkout at build time)."""
import pytest
import torch

import oracle

needs_ref = pytest.mark.skipif(oracle.ref_lib() is None, reason="oracle/_ref was not built")


@needs_ref
@pytest.mark.parametrize("seed,n,gmin,vs,gs", [
    (0, 20000, [-10.0, -10.0, -10.0], 0.05, [128, 128, 128]),
    (1, 5000, [-2.0, -1.5, -1.0], 0.1, [40, 30, 20]),
    (2, 3000, [0.0, 0.0, 0.0], 0.3, [7, 11, 5]),
])
def test_counts_and_occupancy_equal_header(seed, n, gmin, vs, gs):
    g = torch.Generator().manual_seed(seed)
    span = torch.tensor([gs[0] * vs, gs[1] * vs, gs[2] * vs])
    pts = torch.rand(n, 3, generator=g) * span * 1.5 + torch.tensor(gmin) - 0.25 * span
    dens = oracle.ref_header_voxelize(pts, gmin, vs, gs, density=True)
    occ = oracle.ref_header_voxelize(pts, gmin, vs, gs, density=False)
    counts = oracle.voxelize_pointcloud(pts, None, gmin, vs, gs, "count").flatten()
    mine_occ = oracle.voxelize_pointcloud(pts, None, gmin, vs, gs, "occupancy").flatten()
    assert torch.equal(counts.float(), dens)
    assert torch.equal(mine_occ.float(), occ)


@needs_ref
def test_header_resample_is_a_different_algorithm():
    """The header's resampler brackets with <= and has no epsilon: it is not the parity target.
    This documents the divergence (values differ, shapes agree) so nobody swaps oracles by accident."""
    import ctypes
    g = torch.Generator().manual_seed(0)
    B, S, T, D = 2, 50, 40, 4
    st = torch.sort(torch.rand(B, S, generator=g), dim=1).values.contiguous()
    tt = torch.sort(torch.rand(B, T, generator=g), dim=1).values.contiguous()
    src = torch.randn(B, S, D, generator=g)
    out = torch.empty(B, T, D)
    oracle.ref_lib().ref_resample_f32(src.data_ptr(), st.data_ptr(), tt.data_ptr(), out.data_ptr(), B, S, T, D)
    mine = oracle.resample_trajectories(src, st, tt)
    assert torch.allclose(out, mine, atol=1e-3)          # same interpolation up to rounding / ties
    assert not torch.equal(out, mine)                    # but not the same arithmetic
