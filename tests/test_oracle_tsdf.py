"""Known answers for the oracle's truncated-signed-distance restatement (the reference holds no vectors for it):
values a reader can verify by hand from the kernel's rule (point_cloud_voxelization.cu:326-373)."""
import numpy as np

from oracle import tsdf as otsdf


def test_single_point_on_a_voxel_centre():
    # 5^3 grid of unit voxels from the origin; the point sits on the centre of voxel (z=2, y=2, x=2)
    pts = np.array([[[2.5, 2.5, 2.5]]], dtype=np.float32)
    t, w = otsdf.voxelize_tsdf(pts, None, (5, 5, 5), 1.0, (0.0, 0.0, 0.0), 1.5)
    assert t.shape == (1, 5, 5, 5) and w.shape == t.shape
    assert t[0, 2, 2, 2] == 0.0 and w[0, 2, 2, 2] == 1.0
    # face neighbours are 1 voxel away: 1 / 1.5; edge neighbours sqrt(2) / 1.5; corners sqrt(3) > 1.5 untouched
    assert t[0, 2, 2, 3] == np.float32(1.0) * (np.float32(1.0) / np.float32(1.5))
    assert t[0, 1, 2, 2] == t[0, 2, 2, 3] == t[0, 2, 3, 2]
    assert t[0, 2, 3, 3] == np.sqrt(np.float32(2.0)) * (np.float32(1.0) / np.float32(1.5))
    assert t[0, 3, 3, 3] == 0.0 and w[0, 3, 3, 3] == 0.0
    assert w.sum() == 1 + 6 + 12


def test_sign_follows_the_closest_points_normal():
    # surface point at x = 2.5 with its normal towards +x: centres at larger x are in front (dot > 0 -> negative per the
    # kernel's rule "dot(normal, centre - point) > 0 -> -dist"), centres at smaller x positive
    pts = np.array([[[2.5, 0.5, 0.5]]], dtype=np.float32)
    nrm = np.array([[[1.0, 0.0, 0.0]]], dtype=np.float32)
    t, w = otsdf.voxelize_tsdf(pts, nrm, (1, 1, 5), 1.0, (0.0, 0.0, 0.0), 2.5)
    row = t[0, 0, 0]
    assert row[2] == 0.0
    assert row[3] == -np.float32(1.0) * (np.float32(1.0) / np.float32(2.5)) and row[4] < row[3] < 0
    assert row[1] == -row[3] and row[0] == -row[4]
    assert (w[0, 0, 0] == 1.0).all()


def test_closest_point_wins_and_weights_count_points():
    pts = np.array([[[0.5, 0.5, 0.5], [2.5, 0.5, 0.5], [np.nan, 0.0, 0.0]]], dtype=np.float32)
    t, w = otsdf.voxelize_tsdf(pts, None, (1, 1, 3), 1.0, (0.0, 0.0, 0.0), 1.25)
    inv = np.float32(1.0) / np.float32(1.25)
    assert list(t[0, 0, 0]) == [0.0, np.float32(1.0) * inv, 0.0]
    assert list(w[0, 0, 0]) == [1.0, 2.0, 1.0]
