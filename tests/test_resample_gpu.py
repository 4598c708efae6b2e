"""Parity of the CUDA resampler (through the C ABI / Python operator) with the CPU oracle.
Gates: bracket rows exact; fp32 values bit-exact (stronger than rel 1e-6); bf16 values equal to the
oracle's fp32 result rounded once to bf16 (0 ulp, inside the 1-ulp allowance)."""
import pytest
import torch

import oracle
import robocache
from conftest import bits, golden_names, load_golden
from robogoat_b200 import ops
import workloads

pytestmark = [pytest.mark.gpu, pytest.mark.usefixtures("kernel_choice")]
DEV = "cuda:0"


def expected(src, st, tt):
    ref = oracle.resample_trajectories(src, st, tt)
    return oracle.round_to_bf16(ref) if src.dtype == torch.bfloat16 else ref


def run(src, st, tt):
    out = robocache.resample_trajectories(src.to(DEV), st.to(DEV), tt.to(DEV))
    torch.cuda.synchronize()
    return out.cpu()


def assert_exact(out, exp, what=""):
    assert out.shape == exp.shape and out.dtype == exp.dtype
    same = bits(out) == bits(exp)
    if not bool(same.all()):
        # NaN payloads may differ; everything else must match bit for bit
        both_nan = torch.isnan(out.float()) & torch.isnan(exp.float())
        bad = ~(same | both_nan)
        assert not bool(bad.any()), f"{what}: {int(bad.sum())} of {bad.numel()} elements differ, max abs " \
                                    f"{(out.float() - exp.float())[bad].abs().max().item()}"


@pytest.mark.parametrize("name", golden_names("resample_"))
def test_golden_vectors(name, cuda_lib):
    g = load_golden(name)
    out = run(g["src"], g["st"], g["tt"])
    exp = oracle.round_to_bf16(g["out"]) if g["_bf16"] else g["out"]
    assert_exact(out, exp, name)
    left, right, w = ops.resample_brackets_cuda(g["st"].to(DEV), g["tt"].to(DEV))
    assert torch.equal(left.cpu(), g["left"]) and torch.equal(right.cpu(), g["right"])


# shapes of the reference's own CUDA parity test (robocache/tests/test_cuda_correctness.py:17-88)
@pytest.mark.parametrize("B,S,T,D", [(1, 50, 25, 64), (8, 100, 50, 128), (32, 500, 256, 256), (32, 500, 250, 256)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_reference_test_shapes(B, S, T, D, dtype, cuda_lib):
    src, st, tt = workloads.resample_inputs(B, S, D, T, dtype=dtype, irregular_targets=True, seed=B + S)
    assert_exact(run(src, st, tt), expected(src, st, tt))


# every access width (16/8/4/2 bytes), ragged rows, short and long rows, S in {1,2,3}, T in {1, 33, ...}
@pytest.mark.parametrize("B,S,T,D", [
    (3, 1, 5, 4), (2, 2, 7, 3), (2, 3, 1, 1), (5, 17, 40, 12), (4, 9, 33, 7), (2, 64, 65, 8), (3, 31, 97, 588),
    (2, 12, 300, 1024), (1, 500, 250, 2), (7, 5, 31, 6), (2, 40, 64, 520), (1, 3, 1000, 16),
])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_ragged_shapes(B, S, T, D, dtype, cuda_lib):
    g = torch.Generator().manual_seed(B * 1000 + S * 10 + D)
    st = workloads.cumsum_times(B, S, g)
    src = torch.randn(B, S, D, generator=g).to(dtype)
    tt = torch.rand(B, T, generator=g) * 1.4 - 0.2          # unsorted, partly outside the source range
    if S > 2 and T > 2:
        tt[:, 0] = st[:, 1]                                   # exact hits on source timestamps
        tt[:, 1] = st[:, -1]
    assert_exact(run(src, st, tt), expected(src, st, tt))
    left, right, w = ops.resample_brackets_cuda(st.to(DEV), tt.to(DEV))
    el, er, ew = oracle.brackets(st, tt)
    assert torch.equal(left.cpu(), el) and torch.equal(right.cpu(), er)
    assert torch.equal(bits(w), bits(ew))


def test_duplicate_timestamps_and_ties(cuda_lib):
    st = torch.tensor([[0.0, 0.1, 0.1, 0.1, 0.4, 0.4, 0.9, 1.0]]).repeat(3, 1)
    tt = torch.tensor([[0.1, 0.4, 0.0, 1.0, 0.25, 0.9, 0.95, -1.0, 2.0, 0.1000001]]).repeat(3, 1)
    src = torch.randn(3, 8, 20)
    assert_exact(run(src, st, tt), expected(src, st, tt))


def test_unaligned_views_take_the_narrow_path(cuda_lib):
    """Slices that break 16-byte alignment must still be exact (the wrapper makes them contiguous,
    the C ABI picks a narrower access width for odd base addresses)."""
    src, st, tt = workloads.resample_inputs(4, 30, 40, 20, dtype=torch.bfloat16, irregular_targets=True, seed=5)
    s = src[:, :, 1:39]                                      # D=38, non-contiguous
    assert_exact(run(s, st, tt), expected(s.contiguous(), st, tt))
    L = cuda_lib
    # raw C-ABI call on a buffer offset by one element: base pointer only 2-byte aligned
    flat = torch.empty(4 * 30 * 40 + 1, dtype=torch.bfloat16, device=DEV)
    flat[1:] = src.flatten().to(DEV)
    out = torch.empty(4 * 20 * 40 + 1, dtype=torch.bfloat16, device=DEV)
    std, ttd = st.to(DEV), tt.to(DEV)
    rc = L.rc_resample(flat.data_ptr() + 2, std.data_ptr(), ttd.data_ptr(), out.data_ptr() + 2, 4, 30, 20, 40, 1, 0,
                       torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert_exact(out[1:].view(4, 20, 40).cpu(), expected(src, st, tt))
    # a pointer that is not even element aligned is rejected, not dereferenced
    assert L.rc_resample(flat.data_ptr() + 1, std.data_ptr(), ttd.data_ptr(), out.data_ptr(), 4, 30, 20, 40, 1, 0,
                         None) == 4


def test_long_rows_search_global_memory(cuda_lib):
    """S beyond the shared-memory staging limit switches to the global-memory search."""
    B, S, T, D = 2, 60000, 300, 8
    src, st, tt = workloads.resample_inputs(B, S, D, T, irregular_targets=True, seed=11)
    assert_exact(run(src, st, tt), expected(src, st, tt))


def test_dtype_and_shape_errors(cuda_lib):
    src, st, tt = workloads.resample_inputs(2, 10, 8, 5)
    with pytest.raises(RuntimeError, match="Unsupported dtype"):
        robocache.resample_trajectories(src.half().to(DEV), st.to(DEV), tt.to(DEV))
    with pytest.raises(RuntimeError, match="Source length mismatch"):
        robocache.resample_trajectories(src.to(DEV), st[:, :5].to(DEV), tt.to(DEV))
    with pytest.raises(RuntimeError, match="Batch size mismatch"):
        robocache.resample_trajectories(src.to(DEV), st.to(DEV), tt[:1].to(DEV))
    with pytest.raises(RuntimeError, match="3D"):
        robocache.resample_trajectories(src[0].to(DEV), st.to(DEV), tt.to(DEV))
    out = robocache.resample_trajectories(src.to(DEV), st.double().to(DEV), tt.double().to(DEV))   # times in any float dtype
    assert_exact(out.cpu(), expected(src, st, tt))
    empty = robocache.resample_trajectories(src.to(DEV), st.to(DEV), tt[:, :0].to(DEV))
    assert empty.shape == (2, 0, 8)


def test_device_argument_and_identity(cuda_lib):
    src, st, tt = workloads.resample_inputs(4, 50, 16, 50)
    out = robocache.resample_trajectories(src, st, st, device=DEV)       # CPU tensors moved by device=
    assert out.is_cuda and (out.cpu() - src).abs().max() < 1e-5         # robocache/tests/test_trajectory.py:40-53


def test_full_size_properties(cuda_lib):
    """Headline size (B=4096, S=500, D=256, T=250, bf16): checked through properties that do not need
    the oracle on 1.5 GB — a seeded slice against the oracle, exact reproduction of source rows at
    source timestamps, constant rows staying constant, and run-to-run determinism."""
    B, S, D, T = 4096, 500, 256, 250
    src, st, tt = workloads.resample_inputs(B, S, D, T, dtype=torch.bfloat16, irregular_targets=True, seed=0, device=DEV)
    out = robocache.resample_trajectories(src, st, tt)
    out2 = robocache.resample_trajectories(src, st, tt)
    assert torch.equal(out.view(torch.int16), out2.view(torch.int16))
    for sl in (slice(0, 8), slice(2048, 2056), slice(4088, 4096)):
        assert_exact(out[sl].cpu(), expected(src[sl].cpu(), st[sl].cpu(), tt[sl].cpu()), f"slice {sl}")
    # resampling at the source timestamps themselves returns the source rows (weights are 0 or 1 up to
    # the 1e-8 epsilon, far below bf16 resolution)
    ident = robocache.resample_trajectories(src[:64], st[:64], st[:64])
    assert (ident.float() - src[:64].float()).abs().max().item() <= 2 ** -7 * src[:64].float().abs().max().item()
    const = torch.full((16, S, D), 3.0, dtype=torch.bfloat16, device=DEV)
    assert torch.equal(robocache.resample_trajectories(const, st[:16], tt[:16]), torch.full((16, T, D), 3.0, dtype=torch.bfloat16, device=DEV))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_host_buffer_pipeline_matches_device_api(dtype, cuda_lib):
    """The chunked host-buffer entry point (upload / kernel / download overlapped on three streams)
    returns exactly what the device-tensor operator returns, for ragged chunk counts and repeated calls."""
    from robogoat_b200.host_pipeline import resample_trajectories_host
    src, st, tt = workloads.resample_inputs(B=37, S=120, D=64, T=45, dtype=dtype, irregular_targets=True, seed=21)
    exp = expected(src, st, tt)
    for chunk in (5, 8, 37, 100):
        got = resample_trajectories_host(src.pin_memory(), st.pin_memory(), tt.pin_memory(), chunk_rows=chunk)
        assert not got.is_cuda and got.is_pinned()
        assert_exact(got, exp, f"chunk={chunk}")
    out = torch.empty_like(exp).pin_memory()
    src2, st2, tt2 = workloads.resample_inputs(B=37, S=120, D=64, T=45, dtype=dtype, irregular_targets=True, seed=22)
    resample_trajectories_host(src2, st2, tt2, out=out, chunk_rows=6)          # pageable inputs, same cached buffers
    assert_exact(out, expected(src2, st2, tt2), "second call")
    with pytest.raises(RuntimeError, match="CPU tensors"):
        resample_trajectories_host(src.to(DEV), st, tt)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("D", [256, 12])
def test_ragged_items_equal_per_item_oracle_and_last_step_padding(dtype, D, cuda_lib):
    """Variable-length items packed back to back: every item must equal the oracle run on that item alone,
    and the whole batch must equal 'pad with the last step, then resample' (the reference loader's padding,
    robocache/python/robocache/datasets/rtx_loader.py:214-221)."""
    g = torch.Generator().manual_seed(31 + D)
    lens = [1, 2, 3, 17, 500, 64, 0, 129]
    T = 70
    rows, times = [], []
    for n in lens:
        rows.append(torch.randn(n, D, generator=g).to(dtype))
        times.append(workloads.cumsum_times(1, n, g)[0] if n > 0 else torch.empty(0))
    tt = torch.rand(len(lens), T, generator=g) * 1.3 - 0.15
    offs = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int64)
    out = ops.resample_ragged_cuda(torch.cat(rows).to(DEV), torch.cat(times).to(DEV), offs.to(DEV), tt.to(DEV)).cpu()
    for b, n in enumerate(lens):
        if n == 0:
            assert bool((out[b].float() == 0).all())
            continue
        exp = expected(rows[b].unsqueeze(0), times[b].unsqueeze(0), tt[b:b + 1])
        assert_exact(out[b:b + 1], exp, f"item {b} (len {n})")
    # padded batch through the dense operator
    S = max(lens)
    keep = [b for b, n in enumerate(lens) if n > 0]
    pad_rows = torch.stack([torch.cat([rows[b], rows[b][-1:].expand(S - lens[b], -1)]) for b in keep])
    pad_times = torch.stack([torch.cat([times[b], times[b][-1:].expand(S - lens[b])]) for b in keep])
    dense = robocache.resample_trajectories(pad_rows.to(DEV), pad_times.to(DEV), tt[keep].to(DEV)).cpu()
    assert_exact(out[keep], dense, "ragged vs last-step padding")


def test_ragged_bound_below_an_item_length_truncates_the_item(cuda_lib):
    """``max_len`` sizes the staged timestamp row.  A bound smaller than an item must cut that item to its first
    ``max_len`` rows (the result of resampling the truncated item), never read or write past the staging."""
    g = torch.Generator().manual_seed(5)
    lens, bound, T, D = [40, 9, 25], 16, 33, 24
    rows = [torch.randn(n, D, generator=g) for n in lens]
    times = [workloads.cumsum_times(1, n, g)[0] for n in lens]
    tt = torch.rand(len(lens), T, generator=g)
    offs = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int64)
    out = ops.resample_ragged_cuda(torch.cat(rows).to(DEV), torch.cat(times).to(DEV), offs.to(DEV), tt.to(DEV),
                                   max_len=bound).cpu()
    for b, n in enumerate(lens):
        m = min(n, bound)
        exp = expected(rows[b][:m].unsqueeze(0), times[b][:m].unsqueeze(0), tt[b:b + 1])
        assert_exact(out[b:b + 1], exp, f"item {b} (len {n}, bound {bound})")
    # offsets that do not ascend give an empty item (zeros), not a negative length
    bad = offs.clone(); bad[2] = bad[1] - 3
    out = ops.resample_ragged_cuda(torch.cat(rows).to(DEV), torch.cat(times).to(DEV), bad.to(DEV), tt.to(DEV), max_len=64).cpu()
    assert bool((out[1] == 0).all())
    torch.cuda.synchronize()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_bulk_copy_staging_of_time_rows_gives_the_same_bits(dtype, cuda_lib):
    """RC_OPT_GATHER_BULK_STAGE: the gather kernel's timestamp rows staged by bulk asynchronous copies (S a multiple of 4,
    so every row is a whole number of 16-byte pieces) and by ordinary loads, both against the oracle; rows that do not
    qualify for the bulk copy (S = 501) too."""
    from robogoat_b200 import _lib
    cuda_lib.rc_set_option(_lib.OPT_BLOCK_KERNEL, 0)
    try:
        for staged in (1, 0):
            cuda_lib.rc_set_option(_lib.OPT_GATHER_BULK_STAGE, staged)
            for S in (500, 501, 4):
                src, st, tt = workloads.resample_inputs(B=70, S=S, D=256, T=250, dtype=dtype, irregular_targets=True, seed=S)
                out = robocache.resample_trajectories(src.to(DEV), st.to(DEV), tt.to(DEV))
                torch.cuda.synchronize()
                assert_exact(out.cpu(), expected(src, st, tt), f"S={S} bulk staging {staged}")
    finally:
        cuda_lib.rc_set_option(_lib.OPT_GATHER_BULK_STAGE, 1)
        cuda_lib.rc_set_option(_lib.OPT_BLOCK_KERNEL, 1)


def test_gather_kernel_survives_a_bulk_copy_wait_that_runs_out(cuda_lib):
    """The row-gather kernel stages its timestamp rows by bulk copy; with the wait limit at 0 polls every CTA gives up at
    once, counts the event, fetches the rows with ordinary loads and still returns the oracle's bits - nothing on the GPU
    goes wrong in this test."""
    from conftest import DELIBERATE_BULK_TIMEOUTS, bulk_wait_timeouts
    from robogoat_b200 import _lib
    before = bulk_wait_timeouts(cuda_lib)
    assert before == DELIBERATE_BULK_TIMEOUTS[0]
    src, st, tt = workloads.resample_inputs(B=40, S=500, D=256, T=250, dtype=torch.bfloat16, irregular_targets=True, seed=8)
    exp = expected(src, st, tt)
    cuda_lib.rc_set_option(_lib.OPT_BLOCK_KERNEL, 0)
    cuda_lib.rc_set_option(_lib.OPT_BULK_WAIT_LIMIT, 0)
    try:
        out = robocache.resample_trajectories(src.to(DEV), st.to(DEV), tt.to(DEV))
        torch.cuda.synchronize()
    finally:
        cuda_lib.rc_set_option(_lib.OPT_BULK_WAIT_LIMIT, -1)
        cuda_lib.rc_set_option(_lib.OPT_BLOCK_KERNEL, 1)
        after = bulk_wait_timeouts(cuda_lib)
        DELIBERATE_BULK_TIMEOUTS[0] = after
    assert_exact(out.cpu(), exp)
    assert after >= before + 40                       # at least one CTA per batch row gave up
    out = robocache.resample_trajectories(src.to(DEV), st.to(DEV), tt.to(DEV))
    assert_exact(out.cpu(), exp)
    assert bulk_wait_timeouts(cuda_lib) == after      # built-in limit again: no new events


def test_expanded_and_strided_time_rows_are_used_in_place(cuda_lib):
    """Timestamps given as stride-0 expanded rows (the reference's usual linspace(...).expand(B, -1)) or as
    row-strided views give the same bits as their materialised copies."""
    B, S, T, D = 6, 40, 25, 32
    g = torch.Generator().manual_seed(77)
    src = torch.randn(B, S, D, generator=g).to(DEV)
    st_row = torch.sort(torch.rand(S, generator=g)).values.to(DEV)
    tt_row = (torch.rand(T, generator=g) * 1.2 - 0.1).to(DEV)
    st_e, tt_e = st_row.unsqueeze(0).expand(B, -1), tt_row.unsqueeze(0).expand(B, -1)
    ref = robocache.resample_trajectories(src, st_e.contiguous(), tt_e.contiguous())
    assert torch.equal(robocache.resample_trajectories(src, st_e, tt_e), ref)
    assert torch.equal(robocache.resample_trajectories(src, st_e, tt_e.contiguous()), ref)
    wide_st = torch.zeros(B, S + 7, device=DEV); wide_st[:, :S] = st_e
    wide_tt = torch.zeros(B, T + 3, device=DEV); wide_tt[:, :T] = tt_e
    assert torch.equal(robocache.resample_trajectories(src, wide_st[:, :S], wide_tt[:, :T]), ref)   # row stride > row length
    fa = [x.to(DEV) for x in workloads.fusion_inputs(B=B, dtype=torch.float32, seed=3)]
    lin = torch.linspace(0, 1, 50, device=DEV).unsqueeze(0).expand(B, -1)
    assert torch.equal(robocache.fuse_multimodal(*fa[:6], lin), robocache.fuse_multimodal(*fa[:6], lin.contiguous()))
