"""Parity of the one-launch multimodal fusion with the CPU oracle (bit-exact values, see
test_resample_gpu.py for the gates) plus the reference tests' invariants."""
import pytest
import torch

import oracle
import robocache
from conftest import golden_names, load_golden
from robogoat_b200 import ops
import workloads
from test_resample_gpu import DEV, assert_exact

pytestmark = [pytest.mark.gpu, pytest.mark.usefixtures("kernel_choice")]


def expected(args):
    ref = oracle.fuse_multimodal(*args)
    return oracle.round_to_bf16(ref) if args[0].dtype == torch.bfloat16 else ref


def run(args):
    out = robocache.fuse_multimodal(*[a.to(DEV) for a in args])
    torch.cuda.synchronize()
    return out.cpu()


@pytest.mark.parametrize("name", golden_names("fusion_"))
def test_golden_vectors(name, cuda_lib):
    g = load_golden(name)
    args = (g["s1"], g["t1"], g["s2"], g["t2"], g["s3"], g["t3"], g["tt"])
    exp = oracle.round_to_bf16(g["out"]) if g["_bf16"] else g["out"]
    assert_exact(run(args), exp, name)


@pytest.mark.parametrize("B", [1, 4, 37, 256])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_headline_shape(B, dtype, cuda_lib):
    args = workloads.fusion_inputs(B=B, dtype=dtype, seed=B)
    out = run(args)
    assert out.shape == (B, 50, 588)
    assert_exact(out, expected(args))


@pytest.mark.parametrize("streams,T", [
    (((10, 64), (20, 32), (40, 12)), 15),      # robocache/python/robocache/__init__.py:415-432
    (((5, 10), (5, 20), (5, 30)), 5),          # robocache/tests/test_all_operations.py:128-150
    (((7, 3), (1, 5), (2, 1)), 9),             # odd widths, a one-row stream
    (((30, 512), (100, 64), (200, 12)), 1),
    (((3, 8), (4, 1000), (90, 2)), 130),
    (((600, 16), (2, 16), (33, 16)), 64),
])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_ragged_streams(streams, T, dtype, cuda_lib):
    args = list(workloads.fusion_inputs(B=3, T=T, dtype=dtype, seed=T, streams=streams))
    g = torch.Generator().manual_seed(T)
    args[6] = torch.rand(3, T, generator=g) * 1.2 - 0.1     # unsorted targets, some outside the range
    assert_exact(run(args), expected(args))


def test_concat_order_and_clamp(cuda_lib):
    g = load_golden("fusion_concat_order")
    out = run((g["s1"], g["t1"], g["s2"], g["t2"], g["s3"], g["t3"], g["tt"]))
    assert torch.allclose(out[0, 0, :10], torch.ones(10)) and torch.allclose(out[0, 0, 10:30], torch.ones(20) * 2)
    assert torch.allclose(out[0, 0, 30:], torch.ones(30) * 3)
    g = load_golden("fusion_clamp")    # robocache/tests/test_timestamp_alignment.py:292-338
    out = run((g["s1"], g["t1"], g["s2"], g["t2"], g["s3"], g["t3"], g["tt"]))
    for t in (0, 25, -1):
        assert torch.allclose(out[0, t, :8], torch.full((8,), 10.0), atol=0.1)
        assert torch.allclose(out[0, t, 8:12], torch.full((4,), 20.0), atol=0.1)


def test_errors(cuda_lib):
    a = [x.to(DEV) for x in workloads.fusion_inputs(B=2, dtype=torch.float32)]
    bad = list(a)
    bad[2] = bad[2].bfloat16()
    with pytest.raises(RuntimeError, match="dtypes must match"):      # robocache/tests/test_mixed_precision.py:79
        robocache.fuse_multimodal(*bad)
    bad = list(a)
    bad[0] = bad[0].half(); bad[2] = bad[2].half(); bad[4] = bad[4].half()
    with pytest.raises(RuntimeError, match="Unsupported dtype"):
        robocache.fuse_multimodal(*bad)
    bad = list(a)
    bad[3] = bad[3][:, :50]
    with pytest.raises(RuntimeError, match="stream2_times length mismatch"):
        robocache.fuse_multimodal(*bad)
    bad = list(a)
    bad[4] = bad[4][:1]
    with pytest.raises(RuntimeError, match="Batch size mismatch"):
        robocache.fuse_multimodal(*bad)


def test_determinism_and_n_streams(cuda_lib):
    a = [x.to(DEV) for x in workloads.fusion_inputs(B=64, dtype=torch.bfloat16, seed=9)]
    o1, o2 = robocache.fuse_multimodal(*a), robocache.fuse_multimodal(*a)    # robocache/tests/test_determinism.py:24-55
    assert torch.equal(o1.view(torch.int16), o2.view(torch.int16))
    # fusion == per-stream resampling concatenated; also exercises 1, 2 and 5 streams in one launch
    parts = [robocache.resample_trajectories(a[2 * k], a[2 * k + 1], a[6]) for k in range(3)]
    assert torch.equal(torch.cat(parts, dim=-1).view(torch.int16), o1.view(torch.int16))
    five = ops.fuse_streams_cuda([a[0], a[2], a[4], a[2], a[0]], [a[1], a[3], a[5], a[3], a[1]], a[6])
    assert torch.equal(five.view(torch.int16), torch.cat(parts + [parts[1], parts[0]], dim=-1).view(torch.int16))


def test_throughput_size_properties(cuda_lib):
    """B=16384 headline throughput case: a seeded slice against the oracle and equality with per-stream resampling."""
    a = workloads.fusion_inputs(B=16384, dtype=torch.bfloat16, seed=0, device=DEV)
    out = robocache.fuse_multimodal(*a)
    assert out.shape == (16384, 50, 588)
    for sl in (slice(0, 4), slice(9000, 9004), slice(16380, 16384)):
        cpu_args = [x[sl].cpu() for x in a]
        assert_exact(out[sl].cpu(), expected(cpu_args), f"slice {sl}")
    vis = robocache.resample_trajectories(a[0], a[1], a[6])
    assert torch.equal(vis.view(torch.int16), out[:, :, :512].contiguous().view(torch.int16))


def test_bulk_copy_wait_that_runs_out_falls_back_to_plain_loads(kernel_choice, cuda_lib):
    """Failure detection of the staged kernel, made to happen without anything going wrong on the GPU: with the
    wait limit set to 0 polls every CTA gives up on its bulk copies at once, counts the event, fetches the same
    bytes with ordinary loads and still returns the oracle's bits (then waits for the copies before it exits)."""
    from conftest import DELIBERATE_BULK_TIMEOUTS, bulk_wait_timeouts
    from robogoat_b200 import _lib
    before = bulk_wait_timeouts(cuda_lib)
    assert before == DELIBERATE_BULK_TIMEOUTS[0]
    args = list(workloads.fusion_inputs(B=64, dtype=torch.bfloat16, seed=11))
    exp = expected(args)
    assert cuda_lib.rc_set_option(_lib.OPT_BULK_WAIT_LIMIT, 0) == 0
    try:
        got = run(args)
        got2 = run(args)
    finally:
        assert cuda_lib.rc_set_option(_lib.OPT_BULK_WAIT_LIMIT, -1) == 0
        after = bulk_wait_timeouts(cuda_lib)
        DELIBERATE_BULK_TIMEOUTS[0] = after
    assert_exact(got, exp)
    assert_exact(got2, exp)
    if kernel_choice == "staged-block":
        assert after >= before + 2 * 64                  # at least one CTA per item and call gave up
    else:
        assert after == before                           # the row-gather kernel has no such wait
    assert cuda_lib.rc_set_option(_lib.OPT_BULK_WAIT_LIMIT, -2) != 0
    assert_exact(run(args), exp)                         # built-in limit again: no new events
    assert bulk_wait_timeouts(cuda_lib) == after


def test_no_bulk_copy_wait_ever_ran_out(cuda_lib):
    """The bounded mbarrier wait of the staged kernel is a safety net; outside the test that sets its limit to 0
    it must not have fired."""
    from conftest import DELIBERATE_BULK_TIMEOUTS, bulk_wait_timeouts
    assert bulk_wait_timeouts(cuda_lib) == DELIBERATE_BULK_TIMEOUTS[0]


def test_cuda_graph_replay_matches_direct_calls(cuda_lib):
    """Small-batch latency path: the operator captured into a CUDA graph and replayed on new inputs returns
    the same bits as a direct call (robocache/python/robocache/cuda_graph_cache.py:75-148 is the reference's cache)."""
    from robogoat_b200.graphs import GraphCache
    cache = GraphCache(capacity=2)
    for seed in (1, 2, 3):
        a = [x.to(DEV) for x in workloads.fusion_inputs(B=4, dtype=torch.bfloat16, seed=seed)]
        got = cache.run(robocache.fuse_multimodal, *a).clone()
        assert torch.equal(got.view(torch.int16), robocache.fuse_multimodal(*a).view(torch.int16)), seed
    assert cache.stats() == {"entries": 1, "hits": 2, "misses": 1}
    src, st, tt = (x.to(DEV) for x in workloads.resample_inputs(B=8, S=100, D=64, T=40, irregular_targets=True, seed=4))
    got = cache.run(robocache.resample_trajectories, src, st, tt).clone()
    assert torch.equal(got, robocache.resample_trajectories(src, st, tt))
    assert cache.stats()["entries"] == 2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("streams,T,B", [
    (((30, 512), (100, 64), (200, 12)), 50, 1500),      # headline widths, several CTAs per SM
    (((7, 16), (3, 8), (5, 4)), 9, 2500),               # tiny rows, odd lengths
    (((40, 36), (600, 4), (2, 20)), 33, 1300),          # a long time row
])
def test_many_items(streams, T, B, dtype, cuda_lib):
    """Batches of a few thousand items (several waves of CTAs per SM) against the oracle."""
    args = list(workloads.fusion_inputs(B=B, T=T, dtype=dtype, seed=B + T, streams=streams))
    g = torch.Generator().manual_seed(B)
    args[6] = torch.rand(B, T, generator=g) * 1.2 - 0.1
    assert_exact(run(args), expected(args))
