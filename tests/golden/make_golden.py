"""Generate the golden fixtures in this folder from the reference itself.

Run once, in a container that has the reference checkout (it cannot travel with the
tests):

    python tests/golden/make_golden.py --reference-root /path/to/reference

* ``resample_*.npz`` / ``fusion_*.npz`` hold seeded inputs and the outputs of the
  reference's torch CPU path, imported unmodified from
  ``robocache/python/robocache/ops_fallback.py`` (``_interpolate_stream``,
  ``fuse_multimodal_cpu``), plus the bracket rows its lines 132-137 select.
* ``voxel_*.npz`` hold seeded points and the float occupancy / density grids of the
  reference's C++ header ``robocache/validation/cpu_reference.hpp`` compiled unmodified
  behind ``oracle/ref_shim.cpp``.

Input shapes follow the reference's own tests (cited per case).  bf16 tensors are stored
as their int16 bit patterns.
"""
from __future__ import annotations

import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def _np(t: torch.Tensor) -> np.ndarray:
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy()
    return t.numpy()


def _ref_brackets(st: torch.Tensor, tt: torch.Tensor):
    # the index selection of ops_fallback.py:132-137, kept as its own tensors
    S = st.shape[1]
    right = torch.stack([torch.clamp(torch.searchsorted(st[b], tt[b]), 1, S - 1)
                         for b in range(st.shape[0])])
    left = right - 1
    left = torch.where(left < 0, left + S, left)
    return left.to(torch.int32), right.to(torch.int32)


def cumsum_times(B, S, g):
    inc = torch.rand(B, S, generator=g) + 0.5
    st = inc.cumsum(1)
    return ((st - st[:, :1]) / (st[:, -1:] - st[:, :1])).contiguous()


def resample_cases(g):
    cases = {}
    # robocache/tests/test_trajectory.py:55-71 — hand case
    cases["hand_ramp"] = (torch.tensor([[[0.0], [1.0], [2.0]]]), torch.tensor([[0.0, 0.5, 1.0]]),
                          torch.tensor([[0.0, 0.25, 0.5, 0.75, 1.0]]))
    # robocache/python/robocache/__init__.py:391-397 — self-test case
    cases["selftest"] = (torch.tensor([[[1.0], [2.0], [3.0]]]), torch.tensor([[0.0, 0.5, 1.0]]),
                         torch.tensor([[0.25, 0.75]]))
    # robocache/tests/test_trajectory.py:40-53 — identity
    st = torch.linspace(0, 1, 50).unsqueeze(0).expand(4, -1).contiguous()
    cases["identity"] = (torch.randn(4, 50, 16, generator=g), st, st.clone())
    # robocache/tests/test_trajectory.py:151-166 — irregular sorted times
    cases["irregular"] = (torch.randn(4, 50, 16, generator=g),
                          torch.sort(torch.rand(4, 50, generator=g), dim=1).values.contiguous(),
                          torch.sort(torch.rand(4, 32, generator=g), dim=1).values.contiguous())
    # robocache/tests/test_trajectory.py:168-185 — targets before the first source time
    cases["boundary"] = (torch.randn(2, 5, 4, generator=g),
                         torch.tensor([[0.2, 0.4, 0.6, 0.8, 1.0]]).expand(2, -1).contiguous(),
                         torch.tensor([[0.0, 0.1, 0.3, 0.5, 0.7, 0.9, 1.0]]).expand(2, -1).contiguous())
    # robocache/tests/test_all_operations.py:50-61 — single source row
    cases["single_source"] = (torch.randn(1, 1, 4, generator=g), torch.tensor([[0.0]]),
                              torch.linspace(0, 1, 5).unsqueeze(0))
    # robocache/tests/test_all_operations.py:63-75 — targets outside the source range
    cases["outside_range"] = (torch.randn(1, 5, 4, generator=g),
                              torch.linspace(0.2, 0.8, 5).unsqueeze(0),
                              torch.linspace(0, 1, 10).unsqueeze(0))
    # headline generator (cumsum of U(0.5,1.5), normalised; shared linspace targets), thin D
    cases["cfg1_thin"] = (torch.randn(2, 500, 8, generator=g), cumsum_times(2, 500, g),
                          torch.linspace(0, 1, 250).expand(2, -1).contiguous())
    # same generator, bf16 features, irregular unsorted-in-places targets, odd D
    tt = torch.rand(3, 33, generator=g) * 1.2 - 0.1
    cases["bf16_irregular"] = (torch.randn(3, 20, 24, generator=g).bfloat16(),
                               cumsum_times(3, 20, g), tt)
    # duplicate source timestamps and targets that hit source times exactly
    st = torch.tensor([[0.0, 0.1, 0.1, 0.1, 0.4, 0.4, 0.9, 1.0]]).expand(2, -1).contiguous()
    tt = torch.tensor([[0.1, 0.4, 0.0, 1.0, 0.25, 0.9, 0.95, -1.0, 2.0]]).expand(2, -1).contiguous()
    cases["ties"] = (torch.randn(2, 8, 7, generator=g), st, tt)
    return cases


def fusion_cases(g):
    cases = {}

    def feats(B, n1, n2, n3, d=(512, 64, 12), dtype=torch.float32):
        return [torch.randn(B, n, k, generator=g).to(dtype) for n, k in zip((n1, n2, n3), d)]

    # robocache/tests/test_timestamp_alignment.py:59-114 — non-uniform grids
    B = 4
    vt = torch.tensor([0.0, 0.05, 0.1, 0.15, 0.2, 0.7, 0.8, 0.9, 0.95, 1.0]).expand(B, -1)
    pt = torch.tensor([0.0, 0.1, 0.2, 0.3, 0.4, 0.5, 0.6, 0.7, 0.8, 0.9, 1.0]).expand(B, -1)
    it = torch.tensor([0.0, 0.05, 0.1, 0.2, 0.4, 0.6, 0.8, 0.9, 0.95, 1.0]).expand(B, -1)
    tt = torch.tensor([0.0, 0.12, 0.25, 0.35, 0.5, 0.75, 0.88, 1.0]).expand(B, -1)
    v, p, i = feats(B, 10, 11, 10)
    cases["nonuniform"] = (v, vt, p, pt, i, it, tt)
    # robocache/tests/test_timestamp_alignment.py:173-233 — jittered grids
    def jit(n, amp):
        return (torch.linspace(0, 1, n) + torch.rand(n, generator=g) * 2 * amp - amp).sort()[0].expand(B, -1)
    v, p, i = feats(B, 20, 50, 100, d=(64, 16, 12))
    cases["jittered"] = (v, jit(20, 0.01), p, jit(50, 0.005), i, jit(100, 0.0025),
                         torch.linspace(0, 1, 25).expand(B, -1))
    # robocache/tests/test_timestamp_alignment.py:237-288 — skewed sampling rates
    v, p, i = feats(2, 10, 100, 500, d=(32, 16, 12))
    cases["skewed"] = (v, torch.linspace(0, 1, 10).expand(2, -1), p, torch.linspace(0, 1, 100).expand(2, -1),
                       i, torch.linspace(0, 1, 500).expand(2, -1), torch.linspace(0, 1, 50).expand(2, -1))
    # robocache/tests/test_timestamp_alignment.py:292-338 — clamp outside the source range
    cases["clamp"] = (torch.ones(1, 20, 8) * 10.0, torch.linspace(0.2, 0.8, 20).expand(1, -1),
                      torch.ones(1, 30, 4) * 20.0, torch.linspace(0.3, 0.7, 30).expand(1, -1),
                      torch.ones(1, 40, 2) * 30.0, torch.linspace(0.25, 0.75, 40).expand(1, -1),
                      torch.linspace(0.0, 1.0, 50).expand(1, -1))
    # robocache/tests/test_all_operations.py:128-150 — slice order
    lin = torch.linspace(0, 1, 5).unsqueeze(0)
    cases["concat_order"] = (torch.ones(1, 5, 10), lin, torch.ones(1, 5, 20) * 2, lin,
                             torch.ones(1, 5, 30) * 3, lin, lin)
    # headline fusion shape in bf16 (linspace + N(0,1e-3) jitter, sorted), B=2
    def js(n):
        return torch.sort(torch.linspace(0, 1, n) + torch.randn(2, n, generator=g) * 1e-3, dim=1).values
    v, p, i = feats(2, 30, 100, 200, dtype=torch.bfloat16)
    cases["cfg3_bf16"] = (v, js(30), p, js(100), i, js(200), torch.linspace(0, 1, 50).expand(2, -1))
    return cases


def voxel_cases(g):
    cases = {}
    # robocache/tests/test_voxelize_correctness.py:14-97 — U[-10,10)^3 points, seed-style
    cases["uniform_32"] = (torch.rand(1000, 3, generator=g) * 20 - 10, [-10.0, -10.0, -10.0], 0.625, [32, 32, 32])
    # headline occupancy geometry (only a corner of the cloud is inside the grid), thinned
    cases["corner_128"] = (torch.rand(20000, 3, generator=g) * 20 - 10, [-10.0, -10.0, -10.0], 0.05, [128, 128, 128])
    # non-cubic grid: pins the z-major linearisation
    cases["noncubic"] = (torch.rand(5000, 3, generator=g) * 4 - 2, [-2.0, -1.5, -1.0], 0.1, [40, 30, 20])
    # robocache/tests/test_voxelize_correctness.py:163-180 — three points in one voxel
    cases["three_in_one"] = (torch.tensor([[0.01, 0.01, 0.01], [0.02, 0.02, 0.02], [0.03, 0.03, 0.03]]),
                             [0.0, 0.0, 0.0], 0.1, [16, 16, 16])
    # robocache/tests/test_voxelize_correctness.py:142-157 — everything out of bounds
    cases["all_oob"] = (torch.rand(100, 3, generator=g) + 100.0, [-10.0, -10.0, -10.0], 0.1, [32, 32, 32])
    # points exactly on voxel faces and the grid's outer faces
    edge = torch.tensor([[0.0, 0.0, 0.0], [0.1, 0.2, 0.3], [1.6, 0.0, 0.0], [1.5999999, 0.0, 0.0],
                         [-0.0, 0.5, 0.5], [-1e-9, 0.5, 0.5], [0.7, 0.7, 0.7], [0.30000001, 0.6, 0.9]])
    cases["faces"] = (edge, [0.0, 0.0, 0.0], 0.1, [16, 16, 16])
    return cases


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference-root", default=os.path.abspath(os.path.join(ROOT, "..", "reference")))
    args = ap.parse_args()
    sys.path.insert(0, os.path.join(args.reference_root, "robocache", "python"))
    sys.path.insert(0, ROOT)
    from robocache import ops_fallback as ref  # the reference's own module
    import oracle

    oracle.build(args.reference_root)
    g = torch.Generator().manual_seed(20240607)

    for name, (src, st, tt) in resample_cases(g).items():
        out = ref.resample_single_stream_cpu(src, st, tt)
        left, right = _ref_brackets(st, tt)
        np.savez_compressed(os.path.join(HERE, f"resample_{name}.npz"), src=_np(src), st=_np(st), tt=_np(tt),
                            out=_np(out.float()), left=_np(left), right=_np(right),
                            bf16=np.array(src.dtype == torch.bfloat16))
    for name, c in fusion_cases(g).items():
        c = [x.contiguous() for x in c]
        out = ref.fuse_multimodal_cpu(*c)
        np.savez_compressed(os.path.join(HERE, f"fusion_{name}.npz"), s1=_np(c[0]), t1=_np(c[1]), s2=_np(c[2]),
                            t2=_np(c[3]), s3=_np(c[4]), t3=_np(c[5]), tt=_np(c[6]), out=_np(out.float()),
                            bf16=np.array(c[0].dtype == torch.bfloat16))
    for name, (pts, gmin, vs, gs) in voxel_cases(g).items():
        dens = oracle.ref_header_voxelize(pts, gmin, vs, gs, density=True)
        occ = oracle.ref_header_voxelize(pts, gmin, vs, gs, density=False)
        nz = torch.nonzero(dens).flatten()
        assert torch.equal(torch.nonzero(occ).flatten(), nz)
        np.savez_compressed(os.path.join(HERE, f"voxel_{name}.npz"), pts=_np(pts), gmin=np.array(gmin, np.float32),
                            vs=np.float32(vs), gs=np.array(gs, np.int32), nz=_np(nz),
                            density=_np(dens[nz]), occupancy=_np(occ[nz]))
    print("wrote", len(os.listdir(HERE)) - 1, "fixtures to", HERE)


if __name__ == "__main__":
    main()
