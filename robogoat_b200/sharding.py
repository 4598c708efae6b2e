"""Multi-GPU harness: one process per GPU, ``torch.distributed`` for the plumbing.

* Resampling and fusion shard over independent batch rows: contiguous ceil-div slices of ``B``
  (the rule of robocache/kernels/cutlass/multi_gpu.cuh:344-367).  No collective is needed to
  compute a shard; gathering the outputs is optional.
* Voxelisation shards over points.  Every rank bins its slice into a private full grid, the
  partial grids are combined with one collective — ``MAX`` for occupancy (as
  robocache/tests/test_multi_gpu.py:76 does), ``SUM`` for counts and feature sums — and means are
  normalised after the reduce, each rank on its own slab of voxels when ``slab_normalize`` is set.

The collective helpers only call ``torch.distributed`` and work on any backend (NCCL on GPUs; the
CPU test-suite drives them with gloo).  The ``*_sharded`` operators call the CUDA kernels.
"""
from __future__ import annotations

from typing import Optional, Sequence, Tuple

import torch
import torch.distributed as dist


def world(group=None) -> Tuple[int, int]:
    """(rank, world_size); (0, 1) when no process group is initialised."""
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(group), dist.get_world_size(group)
    return 0, 1


def shard_bounds(n: int, rank: int, world_size: int) -> Tuple[int, int]:
    """Contiguous ceil-div slice [begin, end) of ``n`` items owned by ``rank``; trailing ranks may be empty."""
    if world_size <= 0 or not (0 <= rank < world_size):
        raise ValueError(f"bad rank {rank} for world size {world_size}")
    per = (n + world_size - 1) // world_size
    begin = min(n, rank * per)
    return begin, min(n, begin + per)


def shard_rows(tensors: Sequence[torch.Tensor], rank: int, world_size: int) -> list:
    """The rank's slice of dimension 0 of every tensor (all must share that dimension)."""
    n = tensors[0].shape[0]
    for t in tensors:
        if t.shape[0] != n:
            raise RuntimeError("Batch size mismatch")
    a, b = shard_bounds(n, rank, world_size)
    return [t[a:b] for t in tensors]


def gather_rows(local: torch.Tensor, total_rows: int, group=None) -> torch.Tensor:
    """All-gather of ceil-div row shards back into a [total_rows, ...] tensor on every rank."""
    rank, ws = world(group)
    if ws == 1:
        return local
    per = (total_rows + ws - 1) // ws
    padded = local
    if local.shape[0] < per:  # trailing shards are shorter: pad so every rank sends the same size
        pad = torch.zeros((per - local.shape[0],) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
        padded = torch.cat([local, pad], dim=0)
    out = torch.empty((ws * per,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(out, padded.contiguous(), group=group)
    return out[:total_rows]


def reduce_partial_grids(grid: torch.Tensor, counts: Optional[torch.Tensor], mode: str, group=None) -> None:
    """In-place reduce of per-rank partial voxel grids over the group.

    occupancy: element-wise MAX (union); count: SUM of int32 counts (exact); mean: SUM of the fp32
    feature sums and of the int32 counts (call before normalising); max: element-wise MAX of grids whose
    empty voxels hold -inf (``mask_empty_for_max`` / ``unmask_empty_after_max`` around this call: a rank's
    decoded max grid stores 0.0 for voxels it saw no point in, which would beat a negative maximum
    found by another rank).
    """
    _, ws = world(group)
    if ws == 1:
        return
    if mode == "occupancy":
        dist.all_reduce(grid, op=dist.ReduceOp.MAX, group=group)
    elif mode == "count":
        dist.all_reduce(grid, op=dist.ReduceOp.SUM, group=group)
    elif mode == "mean":
        if counts is None:
            raise RuntimeError("mean mode reduces counts together with the feature sums")
        dist.all_reduce(grid, op=dist.ReduceOp.SUM, group=group)
        dist.all_reduce(counts, op=dist.ReduceOp.SUM, group=group)
    elif mode == "max":
        dist.all_reduce(grid, op=dist.ReduceOp.MAX, group=group)
    else:
        raise RuntimeError(f"Invalid mode: {mode}. Must be 'count', 'occupancy', 'mean', or 'max'")


def mask_empty_for_max(grid: torch.Tensor, occupied: torch.Tensor) -> None:
    """In place: voxels this rank saw no point in (``occupied`` == 0, shaped like the grid without its feature
    axis) become -inf, the neutral element of the MAX reduce that follows."""
    grid.masked_fill_((occupied == 0).unsqueeze(-1), float("-inf"))


def unmask_empty_after_max(grid: torch.Tensor, occupied_any: torch.Tensor) -> None:
    """In place, after the reduce: voxels no rank saw a point in (``occupied_any`` == 0 after its own MAX
    reduce) go back to 0.0, what the single-GPU operator returns for them."""
    grid.masked_fill_((occupied_any == 0).unsqueeze(-1), 0.0)


# ----------------------------------------------------------------------------- sharded operators (CUDA)

def resample_sharded(source_data, source_times, target_times, gather: bool = False, group=None) -> torch.Tensor:
    """Each rank resamples its batch slice of the (replicated or host-resident) inputs.

    Returns the rank's [rows, T, D] shard, or the full [B, T, D] on every rank with ``gather=True``.
    """
    from . import ops
    rank, ws = world(group)
    dev = torch.device("cuda", torch.cuda.current_device())
    src, st, tt = (t.to(dev, non_blocking=True) for t in shard_rows([source_data, source_times, target_times], rank, ws))
    out = ops.resample_trajectories_cuda(src, st, tt)
    return gather_rows(out, source_data.shape[0], group) if gather else out


def fuse_sharded(s1, t1, s2, t2, s3, t3, target_times, gather: bool = False, group=None) -> torch.Tensor:
    """Batch-sharded three-stream fusion; see ``resample_sharded``."""
    from . import ops
    rank, ws = world(group)
    dev = torch.device("cuda", torch.cuda.current_device())
    parts = [t.to(dev, non_blocking=True) for t in shard_rows([s1, t1, s2, t2, s3, t3, target_times], rank, ws)]
    out = ops.fuse_multimodal_cuda(*parts)
    return gather_rows(out, s1.shape[0], group) if gather else out


def reduce_scatter_partial_grids(grid: torch.Tensor, counts: Optional[torch.Tensor], mode: str, group=None):
    """Reduce per-rank partial grids so that every rank ends up with the reduced values of its own slab only
    (voxel ids [rank*V/R, (rank+1)*V/R)): half the traffic of an all-reduce, and the dense grid never has to
    exist reduced on one GPU.  Returns (grid_slab [V/R, ...], counts_slab or None).  V must divide by the group size."""
    rank, ws = world(group)
    V = counts.numel() if counts is not None else (grid.numel() if grid.dim() == 3 else grid.numel() // grid.shape[-1])
    if V % ws != 0:
        raise RuntimeError(f"the grid's {V} voxels do not divide over {ws} ranks")
    flat = grid.reshape(V, -1) if grid.dim() == 4 else grid.reshape(V)
    op = dist.ReduceOp.MAX if mode in ("occupancy", "max") else dist.ReduceOp.SUM
    out = torch.empty((V // ws,) + tuple(flat.shape[1:]), dtype=flat.dtype, device=flat.device)
    dist.reduce_scatter_tensor(out, flat.contiguous(), op=op, group=group)
    cout = None
    if mode == "mean":
        if counts is None:
            raise RuntimeError("mean mode reduces counts together with the feature sums")
        cout = torch.empty(V // ws, dtype=counts.dtype, device=counts.device)
        dist.reduce_scatter_tensor(cout, counts.reshape(V).contiguous(), op=dist.ReduceOp.SUM, group=group)
    return out, cout


def voxelize_sharded_slab(points_local: torch.Tensor, features_local: Optional[torch.Tensor] = None,
                          grid_min=(-10.0, -10.0, -10.0), voxel_size: float = 0.1, grid_size=(128, 128, 128),
                          mode: str = "occupancy", group=None) -> torch.Tensor:
    """Like ``voxelize_sharded`` but the result stays sharded: each rank returns the voxels
    [rank*V/R, (rank+1)*V/R) of the union cloud's grid (for a z-major grid: its block of z-planes), shaped
    [V/R] or [V/R, F].  The partial grids are combined with one reduce-scatter and means are normalised on the
    slab only."""
    from . import ops
    rank, ws = world(group)
    res = ops.voxelize_pointcloud_cuda(points_local, features_local, list(grid_min), float(voxel_size), list(grid_size),
                                       mode, normalize=(ws == 1))
    grid = res[0]
    counts = res[1] if mode == "mean" else None
    V = int(grid_size[0]) * int(grid_size[1]) * int(grid_size[2])
    if ws == 1:
        return grid.reshape(V, -1) if grid.dim() == 4 else grid.reshape(V)
    occ = None
    if mode == "max":       # a rank's empty voxels must not take part in the maximum with their 0.0
        occ = ops.voxelize_pointcloud_cuda(points_local, None, list(grid_min), float(voxel_size), list(grid_size),
                                           "occupancy", occupancy_dtype=torch.uint8)[0]
        mask_empty_for_max(grid, occ)
    slab, cslab = reduce_scatter_partial_grids(grid, counts, mode, group)
    if mode == "mean":
        ops.voxel_normalize_cuda(slab, cslab, 0, cslab.numel())
    if mode == "max":
        occ_slab, _ = reduce_scatter_partial_grids(occ, None, "occupancy", group)
        unmask_empty_after_max(slab, occ_slab)
    return slab


def voxelize_sharded(points_local: torch.Tensor, features_local: Optional[torch.Tensor] = None,
                     grid_min=(-10.0, -10.0, -10.0), voxel_size: float = 0.1, grid_size=(128, 128, 128),
                     mode: str = "occupancy", slab_normalize: bool = False, group=None) -> torch.Tensor:
    """Voxelise a point cloud whose points are spread over the ranks.

    ``points_local`` / ``features_local`` are this rank's points (on its GPU).  Every rank returns the
    grid of the union cloud: occupancy/count bit-identical to a single-GPU run on all points, means
    equal up to fp32 summation order.  With ``slab_normalize`` each rank normalises only its own
    ceil-div slab of voxels and the slabs are all-gathered (less normalisation work per rank).
    """
    from . import ops
    rank, ws = world(group)
    occupancy_dtype = torch.uint8 if (mode == "occupancy" and ws > 1) else torch.int32  # 4x smaller reduce payload
    res = ops.voxelize_pointcloud_cuda(points_local, features_local, list(grid_min), float(voxel_size), list(grid_size),
                                       mode, normalize=(ws == 1), occupancy_dtype=occupancy_dtype)
    grid = res[0]
    counts = res[1] if mode == "mean" else None
    if ws == 1:
        return grid
    occ = None
    if mode == "max":       # a rank's empty voxels must not take part in the maximum with their 0.0
        occ = ops.voxelize_pointcloud_cuda(points_local, None, list(grid_min), float(voxel_size), list(grid_size),
                                           "occupancy", occupancy_dtype=torch.uint8)[0]
        mask_empty_for_max(grid, occ)
    reduce_partial_grids(grid, counts, mode, group)
    if mode == "max":
        reduce_partial_grids(occ, None, "occupancy", group)
        unmask_empty_after_max(grid, occ)
    if mode == "occupancy":
        return grid.to(torch.int32)
    if mode == "mean":
        V = counts.numel()
        if slab_normalize:
            a, b = shard_bounds(V, rank, ws)
            ops.voxel_normalize_cuda(grid, counts, a, b)
            F = grid.shape[-1]
            flat = grid.view(V, F)
            full = gather_rows(flat[a:b], V, group)
            return full.view(grid.shape)
        ops.voxel_normalize_cuda(grid, counts, 0, V)
    return grid


# ----------------------------------------------------------------------------- point exchange (all-to-all)

def exchange_buckets(buckets: Sequence[torch.Tensor], send_counts: Sequence[int], group=None,
                     recv_counts: Optional[Sequence[int]] = None):
    """All-to-all of per-destination buckets.

    Every tensor in ``buckets`` holds, along dimension 0, ``send_counts[0]`` rows for rank 0, then
    ``send_counts[1]`` rows for rank 1, ...  Returns ``(received, recv_counts)``: for each input tensor the
    rows this rank received (grouped by source rank), and how many came from each rank.  ``recv_counts`` may be
    passed when the caller already knows them (it saves the small all-to-all that asks).
    """
    rank, ws = world(group)
    send_counts = [int(c) for c in send_counts]
    if len(send_counts) != ws:
        raise RuntimeError(f"{len(send_counts)} send counts for a group of {ws} ranks")
    if ws == 1:
        return [b[:send_counts[0]] for b in buckets], send_counts
    if recv_counts is None:                                 # not known yet: ask the senders
        dev = buckets[0].device
        sc = torch.tensor(send_counts, dtype=torch.int64, device=dev)
        rc = torch.empty_like(sc)
        dist.all_to_all_single(rc, sc, group=group)
        recv_counts = rc.tolist()
    recv_counts = [int(c) for c in recv_counts]
    total_in, total_out = sum(recv_counts), sum(send_counts)
    received = []
    for b in buckets:
        out = torch.empty((total_in,) + tuple(b.shape[1:]), dtype=b.dtype, device=b.device)
        dist.all_to_all_single(out, b[:total_out].contiguous(), recv_counts, send_counts, group=group)
        received.append(out)
    return received, recv_counts


def slab_bounds(n_voxels: int, rank: int, world_size: int) -> Tuple[int, int]:
    """Voxel ids [begin, end) owned by ``rank`` when the grid is cut into ceil-div slabs."""
    return shard_bounds(n_voxels, rank, world_size)


_RESIDENT_BYTES = 96 << 20      # accumulators of one scatter pass should stay L2-resident


def sub_parts(n_voxels: int, feature_width: int, world_size: int, mode: str) -> int:
    """How many sub-ranges each rank's slab is cut into so that one sub-range's accumulators fit in L2."""
    if mode == "occupancy":
        return 1
    slab = (n_voxels + world_size - 1) // world_size
    acc = slab * 4 * (1 + feature_width if mode == "mean" else 1)
    return max(1, min(64 // world_size, (acc + _RESIDENT_BYTES - 1) // _RESIDENT_BYTES))


def exchange_plan(counts: Sequence[Sequence[int]], rank: int, per_group: int) -> dict:
    """Bookkeeping of the point exchange from the count matrix ``counts[s][p]`` = points rank ``s`` holds for
    part ``p`` (part = owner * per_group + sub-range).  Returns for ``rank``:

    ``send_counts[d]`` / ``recv_counts[s]``  records sent to rank d / received from rank s;
    ``runs``         (first record, records, sub-range) of every run in this rank's receive buffer, which is
                     laid out source rank by source rank, sub-ranges in order inside;
    ``dest_start[p]`` first slot of this rank's part-p records in the owner's receive buffer;
    ``totals[d]``    records rank d receives in all.
    """
    R, K = len(counts), int(per_group)
    to_owner = [[sum(counts[s][d * K:(d + 1) * K]) for d in range(R)] for s in range(R)]
    runs, off = [], 0
    for s in range(R):
        for k in range(K):
            c = int(counts[s][rank * K + k])
            runs.append((off, c, k))
            off += c
    dest_start = []
    for d in range(R):
        slot = sum(to_owner[s][d] for s in range(rank))
        for k in range(K):
            dest_start.append(slot)
            slot += int(counts[rank][d * K + k])
    return {"send_counts": to_owner[rank], "recv_counts": [to_owner[s][rank] for s in range(R)], "runs": runs,
            "dest_start": dest_start, "totals": [sum(to_owner[s][d] for s in range(R)) for d in range(R)]}


def _gather_counts(part_counts: torch.Tensor, group=None):
    """Every rank's per-part counts as nested lists (the host synchronisation point of the exchange)."""
    _, ws = world(group)
    if ws == 1:
        return [part_counts.tolist()]
    allc = torch.empty((ws,) + tuple(part_counts.shape), dtype=part_counts.dtype, device=part_counts.device)
    dist.all_gather_into_tensor(allc, part_counts.contiguous(), group=group)
    return allc.tolist()


class PointExchange:
    """Receive buffers for the direct form of the point exchange: every rank's partition kernel stores its
    records straight into the owners' buffers over NVLink (no staging copy, no separate all-to-all).

    ``capacity`` is the number of records this rank can receive per call; a call whose count matrix shows that
    some rank would receive more falls back to the all-to-all form on every rank.  Construction and ``close``
    are collective.
    """

    def __init__(self, capacity: int, feature_width: int, group=None):
        from .peer import PeerBuffer
        self.capacity = int(capacity)
        self.feature_width = int(feature_width)
        self.group = group
        dev = torch.device("cuda", torch.cuda.current_device())
        self._token = torch.zeros(1, dtype=torch.int32, device=dev)
        # the batched form runs the stores over NVLink and the owner's accumulation side by side
        self.move_stream = torch.cuda.Stream(dev)
        self.scatter_stream = torch.cuda.Stream(dev, priority=-1)
        self.ids = self.features = None
        error = None
        try:
            self.ids = PeerBuffer(max(16, 4 * self.capacity), dev)
            self.features = PeerBuffer(max(16, 4 * self.capacity * max(1, self.feature_width)), dev)
        except RuntimeError as e:           # allocation failed here: tell everyone before anybody waits on a handle
            error = e
        if not self._everyone(error is None):
            self._drop()
            raise RuntimeError(f"PointExchange: receive buffers could not be allocated on every rank ({error})")
        for buf in (self.ids, self.features):       # one collective per buffer, agreed on before the next
            try:
                buf.connect(group)
            except RuntimeError as e:               # no peer access / IPC not permitted
                error = e
            if not self._everyone(error is None):
                self._drop()
                raise RuntimeError(f"PointExchange: peer buffers could not be mapped on every rank ({error})")

    def _everyone(self, ok: bool) -> bool:
        flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device=self._token.device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
        return bool(flag.item())

    def _drop(self) -> None:
        for b in (self.ids, self.features):
            if b is not None:
                b.close()
        self.ids = self.features = None

    def stream_barrier(self) -> None:
        """Orders, on the current stream, everything the other ranks enqueued before their call of this
        method before everything this rank enqueues after it."""
        dist.all_reduce(self._token, group=self.group)

    def close(self) -> None:
        self._drop()


def bucket_slice_windows(chunks: int, ranks: int, slices: int, s: int):
    """Bookkeeping of the sliced bucket exchange.  Every rank's ``chunks`` blocks of an owner's pool (rank r's start at
    block ``r * chunks``) are cut into ``slices`` runs of ``ceil(chunks / slices)`` blocks; slice ``s`` of the exchange is
    run ``s`` of every rank.  Returns ``(first_chunk, n_chunks, first_blocks)``: the slice's first chunk and chunk count
    inside a rank's cloud (0 chunks for slices beyond the capacity) and, per source rank, the first block of its window
    in the owner's pool."""
    chunks, ranks, slices, s = int(chunks), int(ranks), int(slices), int(s)
    if chunks < 0 or ranks < 1 or slices < 1 or not 0 <= s < slices:
        raise ValueError("bad slice geometry")
    per = (chunks + slices - 1) // slices
    first = min(s * per, chunks)
    n = min(per, chunks - first)
    return first, n, [r * chunks + first for r in range(ranks)]


def sparse_list_offsets(rank: int, ranks: int, capacity: int):
    """Bookkeeping of the sparse reduction's record lists: every rank's pool holds one list of ``capacity`` records per
    source rank, source s at record ``s * capacity``.  Returns ``(others, write_at, read_at)``: the other ranks in the
    order they are served (starting with the neighbour, which spreads the link load), the record offset of this rank's
    list inside every other rank's pool, and the record offsets of the others' lists inside this rank's pool."""
    rank, ranks, capacity = int(rank), int(ranks), int(capacity)
    if not 0 <= rank < ranks or capacity < 0:
        raise ValueError("bad rank or capacity")
    others = [(rank + k) % ranks for k in range(1, ranks)]
    return others, rank * capacity, [s * capacity for s in others]


class BucketExchange:
    """Record pools for the bucket form of the point exchange (mean mode, four feature channels).  A chunk's block in
    a pool has a fixed place and capacity, so the exchange needs no counts, no host synchronisation and no all-to-all -
    only a barrier on the stream before it (everybody has finished with the previous call's records) and after.

    Two transports over the same pools.  ``fetch=False`` (default): the bucket kernel stores each owner's records
    straight into that owner's memory over NVLink and the accumulation reads locally.  ``fetch=True``: every rank buckets
    into its OWN memory, one region per owner, and each owner's accumulation kernel reads its regions of all the ranks'
    pools with plain loads over NVLink as it goes; measured slower (2 GPUs, 2^26 points each: 2.67 ms against 2.50 - the
    accumulation's loads reach 340 GB/s of the link, the bucket kernel's stores 520), kept for hosts where only peer reads
    are possible.

    ``points_per_rank`` is the largest cloud a rank may pass per call; every rank holds
    ``world * ceil(points_per_rank / 1024)`` blocks of about 1 K records of 20 bytes.  Construction and ``close`` are
    collective."""

    def __init__(self, points_per_rank: int, n_voxels: int, group=None, fetch: bool = False,
                 sub_ranges: Optional[int] = None, barrier: str = "peer"):
        from .peer import PeerBuffer, PeerBarrier
        if barrier not in ("peer", "nccl"):
            raise ValueError("barrier must be 'peer' (flag kernel over NVLink) or 'nccl' (4-byte all-reduce)")
        self.barrier = None
        self.group = group
        self.fetch = bool(fetch)
        rank, ws = world(group)
        if ws > 16:
            raise RuntimeError("the bucket exchange supports at most 16 ranks")
        self.rank, self.world = rank, ws
        self.per_group = max(1, min(16 // ws, sub_parts(int(n_voxels), 4, ws, "mean")))
        if sub_ranges is not None:          # fewer sub-ranges: larger pieces on the link, less locality for the owner's atomics
            if not 1 <= int(sub_ranges) <= 16 // ws:
                raise ValueError(f"sub_ranges must be between 1 and {16 // ws} for {ws} ranks")
            self.per_group = int(sub_ranges)
        self.chunks = (int(points_per_rank) + 1023) // 1024
        self.capacity = self.chunks * 1024
        dev = torch.device("cuda", torch.cuda.current_device())
        self.block = int(_lib_handle().rc_voxel_bucket_block_records(self.per_group))
        self.n_blocks = ws * self.chunks
        self._token = torch.zeros(1, dtype=torch.int32, device=dev)
        self.ids = self.features = self.runs = None
        error = None
        try:
            self.ids = PeerBuffer(max(128, self.n_blocks * self.block * 4), dev)
            self.features = PeerBuffer(max(128, self.n_blocks * self.block * 16), dev)
            self.runs = PeerBuffer(max(128, self.per_group * self.n_blocks * 4), dev)
        except RuntimeError as e:
            error = e
        if not self._everyone(error is None):
            self.close()
            raise RuntimeError(f"BucketExchange: record pools could not be allocated on every rank ({error})")
        for buf in (self.ids, self.features, self.runs):
            try:
                buf.connect(group)
            except RuntimeError as e:
                error = e
            if not self._everyone(error is None):
                self.close()
                raise RuntimeError(f"BucketExchange: peer buffers could not be mapped on every rank ({error})")
        if barrier == "peer":
            self.barrier = PeerBarrier(group, dev)

    def _everyone(self, ok: bool) -> bool:
        flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device=self._token.device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
        return bool(flag.item())

    def stream_barrier(self) -> None:
        """Orders, on the current stream, everything the other ranks enqueued before their call of this method
        before everything this rank enqueues after it: a flag kernel over NVLink (``peer.PeerBarrier``, bounded wait)
        or, with ``barrier="nccl"``, a 4-byte all-reduce."""
        if self.barrier is not None:
            self.barrier.wait()
        else:
            dist.all_reduce(self._token, group=self.group)

    def barrier_timed_out(self) -> bool:
        """True if a flag barrier gave up waiting for a rank (the results since then are not to be trusted)."""
        return self.barrier is not None and self.barrier.timed_out()

    def destinations(self):
        """(ids, features, runs, first_block, pool_blocks) for this rank's bucket kernel."""
        if not self.fetch:      # owner d's pool lives in d's memory; this rank's blocks start at rank * chunks
            return self.ids.peers, self.features.peers, self.runs.peers, self.rank * self.chunks, self.n_blocks
        # own memory, region d for owner d: chunks blocks of records and a [per_group][chunks] table each
        rec = self.chunks * self.block
        return ([self.ids.ptr + d * rec * 4 for d in range(self.world)],
                [self.features.ptr + d * rec * 16 for d in range(self.world)],
                [self.runs.ptr + d * self.per_group * self.chunks * 4 for d in range(self.world)], 0, self.chunks)

    def sources(self):
        """(ids, features, runs, blocks_per_source) for this rank's accumulation as an owner."""
        if not self.fetch:
            return [self.ids.ptr], [self.features.ptr], [self.runs.ptr], self.n_blocks
        rec = self.chunks * self.block
        d = self.rank           # region `rank` of every source's pool
        return ([p + d * rec * 4 for p in self.ids.peers], [p + d * rec * 16 for p in self.features.peers],
                [p + d * self.per_group * self.chunks * 4 for p in self.runs.peers], self.chunks)

    def slice_sources(self, s: int, slices: int):
        """(ids, features, runs, blocks) of slice ``s`` for this rank's accumulation: one window per source rank
        inside this rank's pool (storing form only); the run tables keep the pool's row length ``n_blocks``."""
        if self.fetch:
            raise RuntimeError("sliced accumulation is built for the storing form of the bucket exchange")
        _, n, blocks = bucket_slice_windows(self.chunks, self.world, slices, s)
        return ([self.ids.ptr + b * self.block * 4 for b in blocks], [self.features.ptr + b * self.block * 16 for b in blocks],
                [self.runs.ptr + b * 4 for b in blocks], n)

    def streams(self):
        """Side streams of the sliced form: (the slices' barriers, the owner's accumulation), both of default priority
        (with the bucket kernels on a high-priority stream single calls took 11-15 ms instead of 2.4)."""
        if getattr(self, "_streams", None) is None:
            dev = self._token.device
            self._streams = (torch.cuda.Stream(dev), torch.cuda.Stream(dev))
        return self._streams

    def close(self) -> None:
        for b in (self.ids, self.features, self.runs, self.barrier):
            if b is not None:
                b.close()
        self.ids = self.features = self.runs = self.barrier = None


class SparseReduce:
    """Record lists for the sparse reduction of partial grids (mean mode, four feature channels): every rank holds, for
    every source rank, a list of ``records_per_pair`` (voxel id, feature sums, count) records that the source fills
    with plain stores over NVLink.  24 bytes per record; construction and ``close`` are collective."""

    def __init__(self, records_per_pair: int, group=None, barrier: str = "peer"):
        from .peer import PeerBuffer, PeerBarrier
        if barrier not in ("peer", "nccl"):
            raise ValueError("barrier must be 'peer' (flag kernel over NVLink) or 'nccl' (4-byte all-reduce)")
        self.barrier = None
        self.group = group
        rank, ws = world(group)
        if ws > 16:
            raise RuntimeError("the sparse reduction supports at most 16 ranks")
        self.rank, self.world = rank, ws
        self.capacity = int(records_per_pair)
        dev = torch.device("cuda", torch.cuda.current_device())
        self._token = torch.zeros(1, dtype=torch.int32, device=dev)
        self.cursors = torch.zeros(16, dtype=torch.int32, device=dev)
        self.overflow = torch.zeros(1, dtype=torch.int32, device=dev)
        self.ids = self.sums = self.counts = self.nrec = None
        error = None
        try:
            self.ids = PeerBuffer(max(128, ws * self.capacity * 4), dev)
            self.sums = PeerBuffer(max(128, ws * self.capacity * 16), dev)
            self.counts = PeerBuffer(max(128, ws * self.capacity * 4), dev)
            self.nrec = PeerBuffer(128, dev)
        except RuntimeError as e:
            error = e
        if not self._everyone(error is None):
            self.close()
            raise RuntimeError(f"SparseReduce: record lists could not be allocated on every rank ({error})")
        for buf in (self.ids, self.sums, self.counts, self.nrec):
            try:
                buf.connect(group)
            except RuntimeError as e:
                error = e
            if not self._everyone(error is None):
                self.close()
                raise RuntimeError(f"SparseReduce: peer buffers could not be mapped on every rank ({error})")
        if barrier == "peer":
            self.barrier = PeerBarrier(group, dev)

    def _everyone(self, ok: bool) -> bool:
        flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device=self._token.device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
        return bool(flag.item())

    def stream_barrier(self) -> None:
        """As ``BucketExchange.stream_barrier``."""
        if self.barrier is not None:
            self.barrier.wait()
        else:
            dist.all_reduce(self._token, group=self.group)

    def failed(self) -> bool:
        """Collective, synchronises: true on every rank if, since the last call of this method, a record list
        overflowed anywhere or a flag barrier gave up waiting - the slabs computed since are then not to be trusted."""
        flag = self.overflow.clone()
        self.overflow.zero_()                   # a barrier's time-out stays raised: nothing after it can be trusted
        if self.barrier is not None:
            flag |= self.barrier.status
        dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=self.group)
        return bool(int(flag.item()))

    def destinations(self, owners):
        """Addresses of this rank's list in every owner's memory: (ids, sums, counts, nrec)."""
        _, off, _ = sparse_list_offsets(self.rank, self.world, self.capacity)
        return ([self.ids.peers[d] + off * 4 for d in owners], [self.sums.peers[d] + off * 16 for d in owners],
                [self.counts.peers[d] + off * 4 for d in owners], [self.nrec.peers[d] + self.rank * 4 for d in owners])

    def sources(self, sources):
        """Addresses of the lists this rank received from ``sources``: (ids, sums, counts, nrec)."""
        offs = [s * self.capacity for s in sources]
        return ([self.ids.ptr + o * 4 for o in offs], [self.sums.ptr + o * 16 for o in offs],
                [self.counts.ptr + o * 4 for o in offs], [self.nrec.ptr + s * 4 for s in sources])

    def close(self) -> None:
        for b in (self.ids, self.sums, self.counts, self.nrec, self.barrier):
            if b is not None:
                b.close()
        self.ids = self.sums = self.counts = self.nrec = self.barrier = None


class SparseGather:
    """One record list per rank for the replicated form of the sparse reduction: a rank writes the occupied voxels of
    its WHOLE partial grid into its own list (local stores), and every other rank reads that list over NVLink while it
    merges.  ``records_per_rank`` bounds the occupied voxels of one rank's partial grid.  Construction and ``close``
    are collective."""

    def __init__(self, records_per_rank: int, group=None, barrier: str = "peer"):
        from .peer import PeerBuffer, PeerBarrier
        if barrier not in ("peer", "nccl"):
            raise ValueError("barrier must be 'peer' (flag kernel over NVLink) or 'nccl' (4-byte all-reduce)")
        self.group = group
        self.rank, self.world = world(group)
        if self.world > 16:
            raise RuntimeError("the sparse reduction supports at most 16 ranks")
        self.capacity = int(records_per_rank)
        dev = torch.device("cuda", torch.cuda.current_device())
        self._token = torch.zeros(1, dtype=torch.int32, device=dev)
        self.cursors = torch.zeros(16, dtype=torch.int32, device=dev)
        self.overflow = torch.zeros(1, dtype=torch.int32, device=dev)
        self.barrier = None
        self.ids = self.sums = self.counts = self.nrec = None
        error = None
        try:
            self.ids = PeerBuffer(max(128, self.capacity * 4), dev)
            self.sums = PeerBuffer(max(128, self.capacity * 16), dev)
            self.counts = PeerBuffer(max(128, self.capacity * 4), dev)
            self.nrec = PeerBuffer(128, dev)
        except RuntimeError as e:
            error = e
        if not self._everyone(error is None):
            self.close()
            raise RuntimeError(f"SparseGather: record lists could not be allocated on every rank ({error})")
        for buf in (self.ids, self.sums, self.counts, self.nrec):
            try:
                buf.connect(group)
            except RuntimeError as e:
                error = e
            if not self._everyone(error is None):
                self.close()
                raise RuntimeError(f"SparseGather: peer buffers could not be mapped on every rank ({error})")
        if barrier == "peer":
            self.barrier = PeerBarrier(group, dev)

    _everyone = SparseReduce._everyone
    stream_barrier = SparseReduce.stream_barrier
    failed = SparseReduce.failed

    def close(self) -> None:
        for b in (self.ids, self.sums, self.counts, self.nrec, self.barrier):
            if b is not None:
                b.close()
        self.ids = self.sums = self.counts = self.nrec = self.barrier = None


def voxelize_sharded_sparse_full(points_local: torch.Tensor, features_local: Optional[torch.Tensor], exchange: SparseGather,
                                 grid_min=(-10.0, -10.0, -10.0), voxel_size: float = 0.1, grid_size=(128, 128, 128),
                                 mode: str = "mean", check: bool = True):
    """Voxelisation of a cloud spread over the ranks with the FULL grid on every rank - what ``voxelize_sharded`` (dense
    partial grids + NCCL all-reduce, the reference's multi-GPU form) returns - by a sparse all-gather: every rank bins
    its own points into a private full grid, lists that grid's occupied voxels in its own memory, and after a barrier
    merges the other ranks' lists, read over NVLink, into its grid.  ``mode``: "mean" (four feature channels; returns the
    normalised [X,Y,Z,4] grid), "count" or "occupancy" (int32 [X,Y,Z]).  Bytes crossing NVLink: 24 (8 in count and
    occupancy mode) per occupied voxel of every other rank, instead of the whole dense grid several times."""
    from . import ops
    rank, ws = exchange.rank, exchange.world
    gx, gy, gz = (int(v) for v in grid_size)
    V = gx * gy * gz
    if mode not in ("mean", "count", "occupancy"):
        raise RuntimeError(f"Invalid mode: {mode}. The sparse all-gather supports 'mean', 'count' and 'occupancy'")
    if mode == "mean":
        if features_local is None or features_local.shape[1] != 4:
            raise RuntimeError("the sparse reduction takes four feature channels")
        grid, counts = ops.voxelize_pointcloud_cuda(points_local, features_local, list(grid_min), float(voxel_size), list(grid_size),
                                                    "mean", normalize=False)
        gflat, cflat = grid.view(V, 4), counts.view(V)
    else:
        grid = ops.voxelize_pointcloud_cuda(points_local, None, list(grid_min), float(voxel_size), list(grid_size), mode)[0]
        gflat, cflat = None, grid.view(V)
    others = [(rank + k) % ws for k in range(1, ws)]
    exchange.stream_barrier()                   # everybody has finished reading this rank's list of the previous call
    ops.voxel_sparse_send_cuda(gflat, cflat, [(0, V)], exchange.capacity, [exchange.ids.ptr],
                               [exchange.sums.ptr if gflat is not None else None], [exchange.counts.ptr], [exchange.nrec.ptr],
                               exchange.cursors, exchange.overflow)
    exchange.stream_barrier()                   # every rank's list is complete
    ops.voxel_sparse_merge_cuda([exchange.ids.peers[s] for s in others],
                                [exchange.sums.peers[s] if gflat is not None else None for s in others],
                                [exchange.counts.peers[s] for s in others], [exchange.nrec.peers[s] for s in others],
                                exchange.capacity, gflat, cflat, 0, V, overflow=exchange.overflow, occupancy=(mode == "occupancy"))
    if check and exchange.failed():
        raise RuntimeError(f"sparse all-gather: a record list of {exchange.capacity} records overflowed on some rank, or a barrier "
                           f"gave up waiting for a rank")
    return grid


def voxelize_sharded_sparse(points_local: torch.Tensor, features_local: torch.Tensor, exchange: SparseReduce,
                            grid_min=(-10.0, -10.0, -10.0), voxel_size: float = 0.1, grid_size=(128, 128, 128),
                            return_counts: bool = False, check: bool = True, mode: str = "mean"):
    """Mean-mode voxelisation of a cloud spread over the ranks, output slab-sharded ([voxels of this rank's slab, 4], a
    view of this rank's full-size partial grid), by a sparse reduction: every rank bins its own points into a private
    full grid, sends each other rank only the occupied voxels of that rank's slab, and adds what it receives to its own
    slab.  Pays when the ranks' clouds put many points into each occupied voxel (bytes on NVLink: 24 per occupied voxel
    instead of 20 per point); needs the full grid on every rank.  ``check``: wait for the call and raise on every rank if
    a record list overflowed anywhere (the result is then incomplete); with ``check=False`` the caller asks
    ``exchange.failed()`` when it wants to know.
    ``mode="count"``: points per voxel (int32 [voxels of the slab]); the records are then (voxel id, count) only."""
    from . import ops
    rank, ws = exchange.rank, exchange.world
    V = int(grid_size[0]) * int(grid_size[1]) * int(grid_size[2])
    if mode not in ("mean", "count"):
        raise RuntimeError(f"Invalid mode: {mode}. The sparse reduction supports 'mean' and 'count'")
    if mode == "count":
        grid = None
        counts = ops.voxelize_pointcloud_cuda(points_local, None, list(grid_min), float(voxel_size), list(grid_size), "count")[0].view(V)
    else:
        if features_local is None or features_local.shape[1] != 4:
            raise RuntimeError("the sparse reduction takes four feature channels")
        grid, counts = ops.voxelize_pointcloud_cuda(points_local, features_local, list(grid_min), float(voxel_size), list(grid_size),
                                                    "mean", normalize=False)
        grid, counts = grid.view(V, 4), counts.view(V)
    a, b = slab_bounds(V, rank, ws)
    others, _, _ = sparse_list_offsets(rank, ws, exchange.capacity)   # start with the neighbour: spreads the link load
    d_ids, d_sums, d_counts, d_nrec = exchange.destinations(others)
    s_ids, s_sums, s_counts, s_nrec = exchange.sources(others)
    if grid is None:
        d_sums, s_sums = [None] * len(others), [None] * len(others)
    exchange.stream_barrier()                   # everybody has merged the records of the previous call
    ops.voxel_sparse_send_cuda(grid, counts, [slab_bounds(V, d, ws) for d in others], exchange.capacity, d_ids, d_sums, d_counts,
                               d_nrec, exchange.cursors, exchange.overflow)
    exchange.stream_barrier()                   # every list is in place
    ops.voxel_sparse_merge_cuda(s_ids, s_sums, s_counts, s_nrec, exchange.capacity, grid, counts, a, b,
                                overflow=exchange.overflow)       # the owner sees by itself if a source dropped records
    if check and exchange.failed():
        raise RuntimeError(f"sparse reduction: a record list of {exchange.capacity} records overflowed on some rank, or a barrier "
                           f"gave up waiting for a rank")
    if grid is None:
        return counts[a:b]
    return (grid[a:b], counts[a:b]) if return_counts else grid[a:b]


def _lib_handle():
    from . import _lib
    return _lib.load()


def voxelize_sharded_buckets(points_local: torch.Tensor, features_local: torch.Tensor, exchange: BucketExchange,
                             grid_min=(-10.0, -10.0, -10.0), voxel_size: float = 0.1, grid_size=(128, 128, 128),
                             return_counts: bool = False, group=None, slices: Optional[int] = None):
    """Mean-mode voxelisation of a cloud spread over the ranks, output slab-sharded as ``voxelize_sharded_exchange``
    returns it ([voxels of this rank's slab, 4]), by the bucket exchange: one bucket kernel, one barrier, then the
    owner's accumulation (which, in the fetching form, pulls the records over NVLink as it goes) and normalisation -
    nothing on the host waits.

    ``slices`` > 1 (storing form): the cloud is bucketed slice after slice on the calling stream, and while slice
    s+1 is on its way over NVLink the owners already accumulate slice s on a second stream; a third stream carries
    the per-slice barriers so that the bucket kernels follow one another without waiting for them.  Default: four
    slices for exchanges sized for 2^22 points per rank or more (where the overlap pays for the extra launches), else one."""
    from . import ops
    rank, ws = world(group)
    V = int(grid_size[0]) * int(grid_size[1]) * int(grid_size[2])
    if features_local is None or features_local.shape[1] != 4:
        raise RuntimeError("the bucket exchange takes four feature channels")
    if points_local.shape[0] > exchange.capacity:
        raise RuntimeError(f"{points_local.shape[0]} points exceed the exchange's capacity of {exchange.capacity} per rank")
    a, b = slab_bounds(V, rank, ws)
    if slices is None:
        slices = 4 if (exchange.chunks >= 4096 and not exchange.fetch) else 1
    if int(slices) > 1 and not exchange.fetch:
        return _buckets_sliced(points_local, features_local, exchange, list(grid_min), float(voxel_size), list(grid_size),
                               int(slices), a, b, return_counts)
    d_ids, d_feats, d_runs, first_block, pool_blocks = exchange.destinations()
    s_ids, s_feats, s_runs, blocks_per_source = exchange.sources()
    exchange.stream_barrier()                   # everybody is done with the records of the previous call
    ops.voxel_bucket_exchange_cuda(points_local, features_local, list(grid_min), float(voxel_size), list(grid_size), ws,
                                   exchange.per_group, exchange.chunks, first_block, pool_blocks, d_ids, d_feats, d_runs)
    exchange.stream_barrier()                   # every rank's records are in place
    grid, counts = ops.voxel_scatter_buckets_cuda(s_ids, s_feats, s_runs, blocks_per_source, exchange.per_group,
                                                  points_local.device, a, b)
    return (grid, counts) if return_counts else grid


def voxelize_sharded_auto(points_local: torch.Tensor, features_local: torch.Tensor, sparse: SparseReduce, buckets: BucketExchange,
                          grid_min=(-10.0, -10.0, -10.0), voxel_size: float = 0.1, grid_size=(128, 128, 128),
                          return_counts: bool = False):
    """Mean-mode voxelisation with slab output that picks its form by trying: the sparse reduction first, and - if a
    record list overflowed on any rank, i.e. the clouds hold too few points per occupied voxel for it to pay - the
    bucket exchange, which takes any cloud.  The lists' capacity is the switch: ``records_per_pair`` below
    ``points_per_rank / world * 20 / 24`` means the sparse form is only ever used where it moves fewer bytes than the
    exchange.  Costs one host synchronisation per call (the check); returns what the two forms return.  The last form
    used is in ``sparse.last_form`` ("sparse" or "buckets")."""
    try:
        out = voxelize_sharded_sparse(points_local, features_local, sparse, grid_min, voxel_size, grid_size,
                                      return_counts=return_counts, check=True)
        sparse.last_form = "sparse"
        return out
    except RuntimeError as e:
        if "overflowed" not in str(e) or (sparse.barrier is not None and sparse.barrier.timed_out()):
            raise
    sparse.last_form = "buckets"
    return voxelize_sharded_buckets(points_local, features_local, buckets, grid_min, voxel_size, grid_size,
                                    return_counts=return_counts)


def _buckets_sliced(points, feats, exchange: BucketExchange, grid_min, voxel_size, grid_size, slices, a, b, return_counts):
    """The bucket exchange in ``slices`` slices on three streams (see ``voxelize_sharded_buckets``)."""
    from . import ops
    dev = points.device
    ws, rank = exchange.world, exchange.rank
    pts = points.to(torch.float32).contiguous()
    fts = feats.to(torch.float32).contiguous()
    N = pts.shape[0]
    d_ids, d_feats, d_runs, first_block, pool_blocks = exchange.destinations()
    main = torch.cuda.current_stream(dev)
    bar_stream, acc_stream = exchange.streams()
    out = ops.voxel_slab_buffers(b - a, 4, "mean", dev)
    exchange.stream_barrier()                   # everybody is done with the records of the previous call
    start = torch.cuda.Event()
    start.record(main)
    acc_stream.wait_event(start)
    with torch.cuda.stream(acc_stream):         # clear the slab while the first slice is bucketed
        ops.voxel_scatter_buckets_cuda([], [], [], 0, exchange.per_group, dev, a, b, normalize=False, out=out)
    for s in range(slices):
        c0, nchunks, _ = bucket_slice_windows(exchange.chunks, ws, slices, s)
        p0, p1 = min(N, c0 * 1024), min(N, (c0 + nchunks) * 1024)
        ops.voxel_bucket_exchange_cuda(pts[p0:p1], fts[p0:p1], grid_min, voxel_size, grid_size, ws, exchange.per_group,
                                       nchunks, first_block + c0, pool_blocks, d_ids, d_feats, d_runs, ctas_per_sm=2)
        stored = torch.cuda.Event()
        stored.record(main)
        bar_stream.wait_event(stored)
        with torch.cuda.stream(bar_stream):     # every rank's records of slice s are in place
            exchange.stream_barrier()
            arrived = torch.cuda.Event()
            arrived.record(bar_stream)
        acc_stream.wait_event(arrived)
        s_ids, s_feats, s_runs, blocks = exchange.slice_sources(s, slices)
        with torch.cuda.stream(acc_stream):
            ops.voxel_scatter_buckets_cuda(s_ids, s_feats, s_runs, blocks, exchange.per_group, dev, a, b,
                                           normalize=(s == slices - 1), table_row_blocks=exchange.n_blocks,
                                           zero_init=False, out=out)
    done = torch.cuda.Event()
    done.record(acc_stream)
    main.wait_event(done)
    for t in out:                               # used on a side stream: keep the allocator from reusing them early
        t.record_stream(acc_stream)
    return (out[0], out[1]) if return_counts else out[0]


def batched_exchange_plans(counts, rank: int, per_group: int):
    """Bookkeeping of the batched direct exchange from ``counts[s][i][p]`` = points rank ``s`` holds for part ``p`` in
    its batch ``i``.  An owner's receive buffer is laid out batch by batch, inside a batch source rank by source rank,
    sub-ranges in order inside.  Returns ``(plans, totals)``: per batch the ``exchange_plan`` of that batch with
    ``dest_start`` and the runs' first records shifted to the batch's place in the buffers, and the records every rank
    receives over all batches."""
    R, nb = len(counts), len(counts[0])
    totals = [0] * R
    plans = []
    for i in range(nb):
        plan = exchange_plan([counts[s][i] for s in range(R)], rank, per_group)
        base = list(totals)
        plan["dest_start"] = [v + base[p // per_group] for p, v in enumerate(plan["dest_start"])]
        plan["runs"] = [(off + base[rank], c, k) for off, c, k in plan["runs"]]
        totals = [t + u for t, u in zip(totals, plan["totals"])]
        plans.append(plan)
    return plans, totals


def _exchange_direct_batched(points, feats, geom, ws, K, rank, direct, mode, F, a, b, batches, group):
    """Direct point exchange in ``batches`` slices of the local cloud: while the partition kernel stores slice i+1 into
    the owners' buffers (NVLink-bound), the owners accumulate slice i (bound by local atomics) on a second stream.  The
    slices' stores and reads are ordered by one token all-reduce per slice on the storing stream.  Returns the slab, or
    None when some rank's buffer is too small (decided alike on every rank)."""
    from . import ops
    dev = points.device
    N = points.shape[0]
    spans = [shard_bounds(N, i, batches) for i in range(batches)]
    counted = [ops.voxel_partition_count_cuda(points[lo:hi], *geom, ws, K) for lo, hi in spans]
    table = torch.stack([pc for pc, _ in counted])                               # [batches, parts]
    plans, totals = batched_exchange_plans(_gather_counts(table, group), rank, K)   # host sync; also orders this call
    if max(totals) > direct.capacity:                                            # after the owners' previous reads
        return None
    out = ops.voxel_slab_buffers(b - a, F, mode, dev)
    main = torch.cuda.current_stream(dev)
    fork = torch.cuda.Event()
    fork.record(main)
    direct.move_stream.wait_event(fork)
    direct.scatter_stream.wait_event(fork)
    with torch.cuda.stream(direct.scatter_stream):
        for t in out:
            t.zero_()
    dest_ids = [direct.ids.peers[p // K] for p in range(ws * K)]
    dest_f = [direct.features.peers[p // K] for p in range(ws * K)] if feats is not None else None
    for i, ((lo, hi), plan) in enumerate(zip(spans, plans)):
        landed = torch.cuda.Event()
        with torch.cuda.stream(direct.move_stream):
            ops.voxel_partition_move_cuda(points[lo:hi], feats[lo:hi] if feats is not None else None, *geom, ws, K, dest_ids,
                                          dest_f, plan["dest_start"], counted[i][1], remote=True)
            direct.stream_barrier()             # every rank's stores of slice i are done
            landed.record(direct.move_stream)
        with torch.cuda.stream(direct.scatter_stream):
            direct.scatter_stream.wait_event(landed)
            ops.voxel_scatter_runs_cuda(direct.ids.ptr, direct.features.ptr if feats is not None else None, dev, F, a, b,
                                        plan["runs"], K, mode, normalize=(i == batches - 1), out=out)
    main.wait_stream(direct.move_stream)
    main.wait_stream(direct.scatter_stream)
    return out[0]


def voxelize_sharded_exchange(points_local: torch.Tensor, features_local: Optional[torch.Tensor] = None,
                              grid_min=(-10.0, -10.0, -10.0), voxel_size: float = 0.1, grid_size=(128, 128, 128),
                              mode: str = "occupancy", group=None, direct: Optional[PointExchange] = None,
                              batches: int = 1) -> torch.Tensor:
    """Slab-sharded voxelisation by exchanging points instead of reducing grids.

    Every rank buckets its points by the rank that owns their voxel (``slab_bounds``) and, inside an owner, by
    L2-sized sub-range of its slab; the buckets travel as 4-byte voxel ids (+ 4*F bytes of features in mean mode)
    and each rank accumulates what it received into its own slab, one sub-range at a time.  Returns the rank's
    slab, shaped [voxels] or [voxels, F] - the same values ``voxelize_sharded_slab`` returns when the voxel count
    divides by the group size - without any rank ever holding the dense grid.  Traffic per rank is
    (R-1)/R * N * (4 + 4F) bytes instead of (R-1)/R of the dense grid.

    Transport: one NCCL all-to-all per tensor by default; with ``direct`` (a ``PointExchange``) the partition
    kernel stores into the owners' receive buffers itself and only two small collectives remain (the count
    matrix, and a barrier between the stores and the owners' reads).  ``batches`` > 1 (direct form only) cuts the
    local cloud into that many slices and overlaps the stores of one slice with the accumulation of the previous.
    """
    from . import ops
    rank, ws = world(group)
    if mode not in ("count", "occupancy", "mean"):
        raise RuntimeError(f"Invalid mode: {mode}. The point exchange supports 'count', 'occupancy' and 'mean'")
    V = int(grid_size[0]) * int(grid_size[1]) * int(grid_size[2])
    feats = features_local if mode == "mean" else None
    if mode == "mean" and feats is None:
        raise RuntimeError("features required for mean/max modes")
    F = feats.shape[1] if feats is not None else 0
    K = sub_parts(V, F, ws, mode)
    geom = (list(grid_min), float(voxel_size), list(grid_size))
    a, b = slab_bounds(V, rank, ws)
    dev = points_local.device
    if direct is not None and ws > 1 and batches > 1 and (feats is None or F == direct.feature_width):
        res = _exchange_direct_batched(points_local, feats, geom, ws, K, rank, direct, mode, F, a, b, int(batches), group)
        if res is not None:
            return res
    elif direct is not None and ws > 1 and (feats is None or F == direct.feature_width):
        part_counts, scratch = ops.voxel_partition_count_cuda(points_local, *geom, ws, K)
        plan = exchange_plan(_gather_counts(part_counts, group), rank, K)       # host sync; also orders this call
        if max(plan["totals"]) <= direct.capacity:                               # after the owners' previous reads
            dest_ids = [direct.ids.peers[p // K] for p in range(ws * K)]
            dest_f = [direct.features.peers[p // K] for p in range(ws * K)] if feats is not None else None
            ops.voxel_partition_move_cuda(points_local, feats, *geom, ws, K, dest_ids, dest_f, plan["dest_start"], scratch,
                                          remote=True)
            direct.stream_barrier()
            res = ops.voxel_scatter_runs_cuda(direct.ids.ptr, direct.features.ptr if feats is not None else None, dev, F,
                                              a, b, plan["runs"], K, mode)
            return res[0]
    ids, fb, part_counts = ops.voxel_partition_cuda(points_local, feats, *geom, ws, K)
    plan = exchange_plan(_gather_counts(part_counts, group), rank, K)            # the host synchronisation of the path
    buckets = [ids] if fb is None else [ids, fb]
    received, _ = exchange_buckets(buckets, plan["send_counts"], group, recv_counts=plan["recv_counts"])
    res = ops.voxel_scatter_runs_cuda(received[0].data_ptr(), received[1].data_ptr() if fb is not None else None, dev, F,
                                      a, b, plan["runs"], K, mode)
    return res[0]
