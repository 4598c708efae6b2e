// Mean-mode voxelisation of large sparse grids by slab-ordered runs.
//
// When the accumulators of a grid (4 + 4F bytes per voxel) do not fit in L2, an atomic that
// misses waits for a DRAM sector and the scatter runs at a fraction of its L2-resident rate.
// This path cuts the voxel ids into P contiguous slabs (blocks of z-planes) and makes every
// slab's atomics one phase of the call:
//
//   bucket kernel   reads points and feature rows once, computes the voxel ids
//                   (robocache/csrc/cuda/voxelize_kernel.cu:43-61), sorts every 1024-point chunk
//                   by slab in shared memory and writes it out as (id, features) records: one
//                   run per slab and chunk, runs padded to 8 records so that every store is a
//                   full sector.  Chunk c owns a fixed block of the record pool, so the layout
//                   does not depend on scheduling and needs no counting pre-pass.
//   scatter kernel  streams the runs slab after slab (sequential reads: no random feature gather) into
//                   atomics that stay inside the current slab
//                   (robocache/csrc/cuda/voxelize_kernel.cu:100-143).
//
// Clearing the grid before and normalising it after are the caller's (rc_voxelize_ex): measured on
// B200, a clear or a normalise interleaved with the atomics costs what it costs alone - requests of
// every kind share the path between the SMs and L2 - so they stay separate, simple passes.
#include "voxel_common.cuh"

namespace rc {
namespace vox {

namespace {

constexpr int kRunPad = 8;                                  // records: 32 bytes of ids, 128 bytes of feature rows
constexpr int kRunChunk = kPointsPerBlock;                  // 1024 points per CTA step
constexpr int kRunBlockMax = kRunChunk + kRunPad * kMeanRunsMaxParts;
constexpr int kBucketStageBytes = kRunBlockMax * 20;        // one sorted chunk: feature rows, then ids
constexpr int kRunLoads = 8;                                // records per lane and step of the scatter: 256 per warp

struct RunRule {
    int P;                  // slabs in use
    unsigned int slab;      // voxel ids per slab, a multiple of 256
    float inv_slab;
    int blk;                // records per chunk block: 1024 + 8 * P
};

// id / slab for quotients below kMeanRunsMaxParts and id < 2^31: float estimate, one correction step either way
__device__ __forceinline__ int slab_of(int id, const RunRule& r) {
    int q = static_cast<int>(__uint2float_rz(static_cast<unsigned int>(id)) * r.inv_slab);
    const unsigned int lo = static_cast<unsigned int>(q) * r.slab;       // q * slab <= id + slab < 2^32
    const unsigned int u = static_cast<unsigned int>(id);
    if (u < lo) --q;
    else if (u - lo >= r.slab) ++q;
    return q;
}

// Multi-GPU form (EXCH): the slabs are grouped by owner - `groups` owners with `per_group` slabs each, slab number
// p = owner * per_group + sub - and every owner has its own record pool and run table, possibly in another GPU's
// memory (plain stores over NVLink; no multicast, nothing is read from a peer).  A pool holds `nblocks` blocks, this
// source's chunk c fills block `block0 + c`, and the owner's segment of the sorted chunk goes to the start of that
// block as one contiguous piece, so every warp store covers whole 128-byte lines up to the segment's tail.
struct ExchangeDest {
    int* ids[kMeanRunsMaxParts];
    float4* feats[kMeanRunsMaxParts];
    unsigned int* runs[kMeanRunsMaxParts];      // [per_group][nblocks] each
    long long block0, nblocks;
    int groups, per_group;
    int bulk_store;                             // 1: segments leave shared memory by bulk asynchronous copies (TMA)
    unsigned int owner_span;                    // voxel ids per owner; RunRule::slab is the span of a slab inside it
    float inv_owner_span;
};

// Bulk asynchronous copy shared memory -> global memory (TMA store, no multicast), tracked by the issuing thread's
// bulk async-group.  A store to a peer GPU issued this way does not hold up the SM's load/store pipeline while NVLink
// is busy, which ordinary stores do - and with them every other CTA of the SM.
__device__ __forceinline__ void bulk_store(void* dst_gmem, const void* src_smem, unsigned int bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                 :: "l"(dst_gmem), "r"(static_cast<unsigned int>(__cvta_generic_to_shared(src_smem))), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// until the copies of this thread's groups have read their shared-memory sources (the data may still be on its way)
__device__ __forceinline__ void bulk_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// the same, but the most recently committed group may still be reading
__device__ __forceinline__ void bulk_store_wait_read_all_but_one() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
__device__ __forceinline__ void fence_async_shared() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Single-GPU form: runs[p * nchunks + c] = (first slot of slab p's run in chunk c's block) << 16 | records in the run.
// Exchange form: the owner's table, runs[sub * nblocks + block0 + c] = (first slot inside the block) << 16 | records.
template <bool EXCH>
__global__ void __launch_bounds__(kThreads, 4)
voxel_bucket_kernel(const float* __restrict__ pts, const float4* __restrict__ feats, long long N, VoxelGeom g,
                    bool pts_aligned, RunRule rule, long long nchunks, unsigned int* __restrict__ runs,
                    int* __restrict__ pool_ids, float4* __restrict__ pool_feats, const __grid_constant__ ExchangeDest dest,
                    const int* __restrict__ gate, int gate_want) {
    __shared__ __align__(16) float s_xyz[kThreads / 32][kPointsPerWarp * 3];
    // the sorted chunk; two of them in the exchange form, so that a CTA can sort its next chunk while the copy engine
    // is still sending the last one over NVLink
    // (dynamic shared memory: kBucketStageBytes per stage, feature rows first)
    extern __shared__ __align__(16) unsigned char s_stage[];
    int stage = 0;
    __shared__ int s_wcnt[kThreads / 32][kMeanRunsMaxParts];
    __shared__ int s_seg[EXCH ? kMeanRunsMaxParts : 1][2];     // first slot and length of every owner's segment
    if (gate != nullptr && *gate != gate_want) return;
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const unsigned int lt_mask = (1u << lane) - 1u;
    const int P = rule.P;
    const int nbits = 32 - __clz(P - 1 > 0 ? P - 1 : 1);
    int* wcnt = s_wcnt[warp];
    if (lane < kMeanRunsMaxParts) wcnt[lane] = 0;
    __syncwarp();
    const long long step = gridDim.x;
    float4 ahead[3];
    {
        const long long base = static_cast<long long>(blockIdx.x) * kRunChunk + warp * kPointsPerWarp;
        if (pts_aligned && blockIdx.x < nchunks && base + kPointsPerWarp <= N) tile_issue(pts, base, lane, ahead);
    }
    for (long long chunk = blockIdx.x; chunk < nchunks; chunk += step) {
        float4* const s_sf = reinterpret_cast<float4*>(s_stage + stage * kBucketStageBytes);
        int* const s_sid = reinterpret_cast<int*>(s_stage + stage * kBucketStageBytes + kRunBlockMax * 16);
        if (EXCH) stage ^= 1;
        const long long base = chunk * kRunChunk + warp * kPointsPerWarp;
        const bool full = base + kPointsPerWarp <= N;
        float4 f[kPointsPerLane];
        const float4* fsrc = feats + base + lane;
#pragma unroll
        for (int i = 0; i < kPointsPerLane; ++i)
            f[i] = (full || base + i * 32 + lane < N) ? __ldcs(fsrc + i * 32) : make_float4(0.f, 0.f, 0.f, 0.f);
        float x[kPointsPerLane], y[kPointsPerLane], z[kPointsPerLane];
        if (pts_aligned && full) {
            float4 now[3] = {ahead[0], ahead[1], ahead[2]};
            const long long nbase = base + step * kRunChunk;
            if (chunk + step < nchunks && nbase + kPointsPerWarp <= N) tile_issue(pts, nbase, lane, ahead);
            tile_unpack(now, s_xyz[warp], lane, x, y, z);
        } else {
            tile_load_slow(pts, base, N, lane, x, y, z);    // points past N come back as NaN and are dropped
        }
        int id[kPointsPerLane], part[kPointsPerLane], rank[kPointsPerLane];
#pragma unroll
        for (int i = 0; i < kPointsPerLane; ++i) {
            id[i] = voxel_id32(x[i], y[i], z[i], g);
            if (EXCH) {
                part[i] = -1;
                if (id[i] >= 0) {
                    const unsigned int u = static_cast<unsigned int>(id[i]);
                    int own = static_cast<int>(__uint2float_rz(u) * dest.inv_owner_span);
                    unsigned int lo = static_cast<unsigned int>(own) * dest.owner_span;
                    if (u < lo) { --own; lo -= dest.owner_span; }
                    else if (u - lo >= dest.owner_span) { ++own; lo += dest.owner_span; }
                    part[i] = own * dest.per_group + slab_of(static_cast<int>(u - lo), rule);
                }
            } else {
                part[i] = (id[i] < 0) ? -1 : slab_of(id[i], rule);
            }
        }
        // rank of every point among the warp's points of the same slab: intersect the ballots of the slab number's
        // bits (__match_any_sync in their place ran 5 % slower, shared-memory atomics on the warp's counters 3 %)
#pragma unroll
        for (int i = 0; i < kPointsPerLane; ++i) {
            unsigned int same = __ballot_sync(0xffffffffu, part[i] >= 0);
#pragma unroll
            for (int bit = 0; bit < 4; ++bit) {
                if (bit < nbits) {
                    const bool on = (part[i] >> bit) & 1;
                    const unsigned int b = __ballot_sync(0xffffffffu, on);
                    same &= on ? b : ~b;
                }
            }
            const unsigned int below = same & lt_mask;
            rank[i] = 0;
            if (part[i] >= 0) rank[i] = wcnt[part[i]] + __popc(below);
            __syncwarp();
            if (part[i] >= 0 && below == 0u) wcnt[part[i]] += __popc(same);
            __syncwarp();
        }
        // the chunk that last used this stage has left shared memory
        if (dest.bulk_store && threadIdx.x < (EXCH ? dest.groups : 1)) {
            if (EXCH) bulk_store_wait_read_all_but_one();
            else bulk_store_wait_read();
        }
        __syncthreads();   // all counts are in; the previous chunk's block has left shared memory
        // every warp derives the layout of the sorted chunk by itself: lane p owns slab p
        int tot = 0, mine = 0;
        if (lane < P) {
#pragma unroll
            for (int w = 0; w < kThreads / 32; ++w) {
                const int t = s_wcnt[w][lane];
                if (w < warp) mine += t;
                tot += t;
            }
        }
        const int padded = (tot + kRunPad - 1) & ~(kRunPad - 1);
        int inc = padded;
#pragma unroll
        for (int off = 1; off < kMeanRunsMaxParts; off <<= 1) {     // lanes past the last slab hold 0
            const int a = __shfl_up_sync(0xffffffffu, inc, off);
            if (lane >= off) inc += a;
        }
        const int total = __shfl_sync(0xffffffffu, inc, kMeanRunsMaxParts - 1);
        const int start = inc - padded;
        const int first = start + mine;
#pragma unroll
        for (int i = 0; i < kPointsPerLane; ++i) {
            const int fi = __shfl_sync(0xffffffffu, first, part[i] & 31);
            if (part[i] >= 0) {
                const int slot = fi + rank[i];
                s_sid[slot] = id[i];
                s_sf[slot] = f[i];
            }
        }
        if (EXCH) {
            // lane p's owner segment starts where the owner's first slab starts
            const int own = lane / dest.per_group;
            const int seg0 = __shfl_sync(0xffffffffu, start, (own * dest.per_group) & 31);
            const int seg1 = __shfl_sync(0xffffffffu, inc, (own * dest.per_group + dest.per_group - 1) & 31);
            if (warp == 0 && lane < P) {
                for (int j = start + tot; j < start + padded; ++j) s_sid[j] = -1;
                dest.runs[own][static_cast<long long>(lane - own * dest.per_group) * dest.nblocks + dest.block0 + chunk] =
                    (static_cast<unsigned int>(start - seg0) << 16) | static_cast<unsigned int>(tot);
                if (lane == own * dest.per_group) { s_seg[own][0] = seg0; s_seg[own][1] = seg1 - seg0; }
            }
        } else if (warp == 0 && lane < P) {
            for (int j = start + tot; j < start + padded; ++j) s_sid[j] = -1;
            runs[static_cast<long long>(lane) * nchunks + chunk] = (static_cast<unsigned int>(start) << 16) | static_cast<unsigned int>(tot);
        }
        if (dest.bulk_store) fence_async_shared();   // this thread's shared-memory writes, for the copy engine
        __syncthreads();
        if (lane < kMeanRunsMaxParts) wcnt[lane] = 0;     // own row, for the next chunk; every warp has read it
        if (EXCH && dest.bulk_store) {
            if (threadIdx.x < dest.groups) {                  // one thread per owner sends that owner's segment
                const int own = threadIdx.x;
                const int s0 = s_seg[own][0], len = s_seg[own][1];     // multiples of 8 records
                const long long o = (dest.block0 + chunk) * rule.blk;
                if (len > 0) {
                    bulk_store(dest.ids[own] + o, s_sid + s0, static_cast<unsigned int>(len) * 4u);
                    bulk_store(dest.feats[own] + o, s_sf + s0, static_cast<unsigned int>(len) * 16u);
                }
                bulk_store_commit();
            }
        } else if (EXCH) {
            for (int own = 0; own < dest.groups; ++own) {
                const int s0 = s_seg[own][0], len = s_seg[own][1];     // multiples of 8 records
                const long long o = (dest.block0 + chunk) * rule.blk;
                int4* dst_i = reinterpret_cast<int4*>(dest.ids[own] + o);
                const int4* src_i = reinterpret_cast<const int4*>(s_sid + s0);
                for (int j = threadIdx.x; j < (len >> 2); j += kThreads) dst_i[j] = src_i[j];
                float4* dst_f = dest.feats[own] + o;
                for (int j = threadIdx.x; j < len; j += kThreads) dst_f[j] = s_sf[s0 + j];
            }
        } else if (dest.bulk_store) {
            if (threadIdx.x == 0) {
                const long long o = chunk * rule.blk;
                if (total > 0) {
                    bulk_store(pool_ids + o, s_sid, static_cast<unsigned int>(total) * 4u);
                    bulk_store(pool_feats + o, s_sf, static_cast<unsigned int>(total) * 16u);
                }
                bulk_store_commit();
            }
        } else {
            const long long o = chunk * rule.blk;
            int4* dst_i = reinterpret_cast<int4*>(pool_ids + o);
            const int4* src_i = reinterpret_cast<const int4*>(s_sid);
            for (int j = threadIdx.x; j < (total >> 2); j += kThreads) __stcs(dst_i + j, src_i[j]);
            float4* dst_f = pool_feats + o;
            for (int j = threadIdx.x; j < total; j += kThreads) __stcs(dst_f + j, s_sf[j]);
        }
    }
    if (dest.bulk_store && threadIdx.x < (EXCH ? dest.groups : 1)) bulk_store_wait_read();   // shared memory must outlive the copies' reads
}

// One slab's runs into the grid (robocache/csrc/cuda/voxelize_kernel.cu:100-143 is the reference's scatter).  A warp
// takes the runs of chunks w, w + warps, ...; up to 256 records of a run are in flight per step, and the next run's
// descriptor is fetched while the current one is accumulated.  One launch per slab: the kernel boundary is what
// keeps the whole GPU on one L2-sized piece of the grid at a time (a single launch walking the slabs in order lets
// the warps drift apart and ran 10 % slower).
__global__ void __launch_bounds__(kThreads)
voxel_run_scatter_kernel(const unsigned int* __restrict__ runs_p, const int* __restrict__ pool_ids,
                         const float4* __restrict__ pool_feats, long long nchunks, int blk, float* __restrict__ grid,
                         int* __restrict__ counts, const int* __restrict__ gate, int gate_want) {
    // The next slab's launch does not depend on this one's results, only on the order: launched as a programmatic
    // dependent it may fill the SMs that this launch's last CTAs leave idle.
    grid_dependency_release();
    if (gate != nullptr && *gate != gate_want) return;
    const int lane = threadIdx.x & 31;
    const long long warps_total = static_cast<long long>(gridDim.x) * (kThreads / 32);
    long long it = static_cast<long long>(blockIdx.x) * (kThreads / 32) + (threadIdx.x >> 5);
    unsigned int desc = (it < nchunks) ? __ldg(runs_p + it) : 0u;
    for (; it < nchunks; it += warps_total) {
        const int n = static_cast<int>(desc & 0xffffu);
        const long long off = it * blk + (desc >> 16);
        const long long next = it + warps_total;
        if (next < nchunks) desc = __ldg(runs_p + next);
        const int* ip = pool_ids + off + lane;
        const float4* fp = pool_feats + off + lane;
        for (int j0 = 0; j0 < n; j0 += 32 * kRunLoads) {
            int id[kRunLoads];
            float4 f[kRunLoads];
#pragma unroll
            for (int i = 0; i < kRunLoads; ++i) {
                const int j = j0 + i * 32 + lane;
                id[i] = -1;
                if (j < n) {
                    id[i] = __ldcs(ip + j0 + i * 32);
                    f[i] = __ldcs(fp + j0 + i * 32);
                }
            }
#pragma unroll
            for (int i = 0; i < kRunLoads; ++i) {
                if (id[i] >= 0) {
                    red_add_v4(grid + static_cast<long long>(id[i]) * 4, f[i]);
                    atomicAdd(counts + id[i], 1);
                }
            }
        }
    }
}

// The owner's side of the bucket exchange: the same accumulation over the blocks of several record pools - one per
// source rank, in this GPU's memory or, when the owner fetches instead of the sources storing, in the sources' memory
// (plain loads over NVLink; no multicast).  Step i takes block i / n of source i % n, so that neighbouring warps
// read from different sources and every link carries its share all the time.
struct ScatterSources {
    const int* ids[kMeanRunsMaxParts];
    const float4* feats[kMeanRunsMaxParts];
    const unsigned int* runs[kMeanRunsMaxParts];    // the current sub-range's row of every source's table
    int n;
};

__global__ void __launch_bounds__(kThreads)
voxel_bucket_scatter_kernel(const __grid_constant__ ScatterSources src, long long blocks, int blk, float* __restrict__ grid,
                            int* __restrict__ counts) {
    grid_dependency_release();      // the next sub-range's launch depends on this one's order only (see voxel_run_scatter_kernel)
    const int lane = threadIdx.x & 31;
    const long long warps_total = static_cast<long long>(gridDim.x) * (kThreads / 32);
    const long long steps = blocks * src.n;
    long long it = static_cast<long long>(blockIdx.x) * (kThreads / 32) + (threadIdx.x >> 5);
    unsigned int desc = (it < steps) ? __ldg(src.runs[it % src.n] + it / src.n) : 0u;
    for (; it < steps; it += warps_total) {
        const int s = static_cast<int>(it % src.n);
        const long long c = it / src.n;
        const int n = static_cast<int>(desc & 0xffffu);
        const long long off = c * blk + (desc >> 16);
        const long long next = it + warps_total;
        if (next < steps) desc = __ldg(src.runs[next % src.n] + next / src.n);
        const int* ip = src.ids[s] + off + lane;
        const float4* fp = src.feats[s] + off + lane;
        for (int j0 = 0; j0 < n; j0 += 32 * kRunLoads) {
            int id[kRunLoads];
            float4 f[kRunLoads];
#pragma unroll
            for (int i = 0; i < kRunLoads; ++i) {
                const int j = j0 + i * 32 + lane;
                id[i] = -1;
                if (j < n) {
                    id[i] = __ldcs(ip + j0 + i * 32);
                    f[i] = __ldcs(fp + j0 + i * 32);
                }
            }
#pragma unroll
            for (int i = 0; i < kRunLoads; ++i) {
                if (id[i] >= 0) {
                    red_add_v4(grid + static_cast<long long>(id[i]) * 4, f[i]);
                    atomicAdd(counts + id[i], 1);
                }
            }
        }
    }
}

long long ceil_div(long long a, long long b) { return (a + b - 1) / b; }
long long round_up(long long a, long long m) { return ceil_div(a, m) * m; }

struct RunsLayout {
    long long nchunks;
    int P;                  // slabs in use
    long long slab;         // voxel ids per slab (multiple of 256)
    int blk;
    uint64_t off_ids, off_feats, total;   // the run table sits at offset 0
};

RunsLayout runs_layout(long long N, long long V, int parts) {
    RunsLayout l{};
    if (parts < 1) parts = 1;
    if (parts > kMeanRunsMaxParts) parts = kMeanRunsMaxParts;
    l.nchunks = ceil_div(N, kRunChunk);
    l.slab = round_up(ceil_div(V, parts), 256);
    l.P = static_cast<int>(ceil_div(V, l.slab));
    l.blk = kRunChunk + kRunPad * l.P;
    const uint64_t table = static_cast<uint64_t>(round_up(static_cast<long long>(l.P) * l.nchunks * 4, 256));
    const uint64_t records = static_cast<uint64_t>(l.nchunks) * static_cast<uint64_t>(l.blk);
    l.off_ids = table;
    l.off_feats = l.off_ids + static_cast<uint64_t>(round_up(static_cast<long long>(records * 4u), 256));
    l.total = l.off_feats + records * 16u;
    return l;
}

}  // namespace

uint64_t mean_runs_scratch_bytes(long long N, long long V, int parts) {
    if (N <= 0 || V <= 0) return 0;
    return runs_layout(N, V, parts).total;
}

int mean_runs_launch(const float* points, const float* features, float* grid, int* counts, long long N,
                     const VoxelGeom& g, long long V, int parts, void* scratch, const int* gate, int gate_want,
                     int device, cudaStream_t st) {
    const RunsLayout l = runs_layout(N, V, parts);
    unsigned char* base = static_cast<unsigned char*>(scratch);
    unsigned int* runs = reinterpret_cast<unsigned int*>(base);
    int* pool_ids = reinterpret_cast<int*>(base + l.off_ids);
    float4* pool_feats = reinterpret_cast<float4*>(base + l.off_feats);
    RunRule rule;
    rule.P = l.P;
    rule.slab = static_cast<unsigned int>(l.slab);
    rule.inv_slab = 1.0f / static_cast<float>(l.slab);
    rule.blk = l.blk;
    const int sms = rc::sm_count(device);
    const long long nb = l.nchunks < 8ll * sms ? l.nchunks : 8ll * sms;
    ExchangeDest none{};
    none.bulk_store = rc::g_bucket_bulk_store.load(std::memory_order_relaxed) ? 1 : 0;
    voxel_bucket_kernel<false><<<static_cast<unsigned int>(nb), kThreads, kBucketStageBytes, st>>>(
        points, reinterpret_cast<const float4*>(features), N, g, rc::aligned_to(points, 16), rule, l.nchunks, runs, pool_ids,
        pool_feats, none, gate, gate_want);
    long long sb = ceil_div(l.nchunks, kThreads / 32);
    if (sb > 8ll * sms) sb = 8ll * sms;
    for (int p = 0; p < l.P; ++p) {
        const unsigned int* runs_p = runs + static_cast<long long>(p) * l.nchunks;
        const int* ids_c = pool_ids;
        const float4* feats_c = pool_feats;
        bool launched = false;
        if (p > 0 && rc::g_scatter_overlap.load(std::memory_order_relaxed)) {   // slab p may start while slab p - 1 drains
            cudaLaunchConfig_t cfg{};
            cfg.gridDim = dim3(static_cast<unsigned int>(sb));
            cfg.blockDim = dim3(kThreads);
            cfg.stream = st;
            cudaLaunchAttribute attr{};
            attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr.val.programmaticStreamSerializationAllowed = 1;
            cfg.attrs = &attr;
            cfg.numAttrs = 1;
            launched = cudaLaunchKernelEx(&cfg, voxel_run_scatter_kernel, runs_p, ids_c, feats_c, l.nchunks, l.blk, grid, counts, gate,
                                          gate_want) == cudaSuccess;
            if (!launched) cudaGetLastError();  // attribute refused: an ordinary launch below
        }
        if (!launched)
            voxel_run_scatter_kernel<<<static_cast<unsigned int>(sb), kThreads, 0, st>>>(runs_p, ids_c, feats_c, l.nchunks, l.blk, grid,
                                                                                       counts, gate, gate_want);
    }
    return rc::check_launch();
}

}  // namespace vox
}  // namespace rc

// ---------------------------------------------------------------- multi-GPU point exchange by buckets
//
// The same two kernels across GPUs, with no counting pass and no host synchronisation: every rank buckets its
// points by (owner, sub-range of the owner's slab) and stores each owner's segment of every chunk straight into
// that owner's record pool (a buffer of the owner's GPU mapped into this process); after a barrier on the stream
// every owner accumulates the blocks it received, sub-range after sub-range.  Because a chunk's block in the pool
// has a fixed place and a fixed capacity (1024 records + padding), nobody needs to know any count in advance.
// No counterpart in the reference, whose multi-GPU test all-reduces dense grids (robocache/tests/test_multi_gpu.py:76).
extern "C" {

using namespace rc::vox;

int32_t rc_voxel_bucket_block_records(int32_t parts_per_group) {
    if (parts_per_group < 1 || parts_per_group > kMeanRunsMaxParts) return 0;
    return static_cast<int32_t>(round_up(kRunChunk + kRunPad * parts_per_group, 32));
}

int rc_voxel_bucket_exchange(const float* points, const float* features, int64_t N, const float grid_min_host[3],
                             float voxel_size, const int32_t grid_size_host[3], int32_t n_groups, int32_t parts_per_group,
                             int64_t chunks, int64_t first_block, int64_t pool_blocks, void* const* dest_ids,
                             void* const* dest_features, void* const* dest_runs, int32_t ctas_per_sm, int device,
                             void* stream) {
    if (grid_min_host == nullptr || grid_size_host == nullptr || dest_ids == nullptr || dest_features == nullptr ||
        dest_runs == nullptr)
        return RC_ERR_NULL_POINTER;
    if (n_groups < 1 || parts_per_group < 1 || N < 0 || chunks < 0 || first_block < 0 || first_block + chunks > pool_blocks)
        return RC_ERR_BAD_SHAPE;
    if (ctas_per_sm < 0 || ctas_per_sm > 8) return RC_ERR_BAD_VALUE;
    if (ctas_per_sm == 0) ctas_per_sm = 8;
    if (static_cast<long long>(n_groups) * parts_per_group > kMeanRunsMaxParts) return RC_ERR_TOO_LARGE;
    if (N > chunks * kRunChunk || N > (1ll << 31) - 4096) return RC_ERR_TOO_LARGE;
    if (!(voxel_size > 0.0f) || !(voxel_size <= 3.0e38f)) return RC_ERR_BAD_VALUE;
    VoxelGeom g;
    g.minx = grid_min_host[0]; g.miny = grid_min_host[1]; g.minz = grid_min_host[2];
    g.vs = voxel_size;
    g.gx = grid_size_host[0]; g.gy = grid_size_host[1]; g.gz = grid_size_host[2];
    if (g.gx < 0 || g.gy < 0 || g.gz < 0) return RC_ERR_BAD_SHAPE;
    if (g.gx >= (1 << 24) || g.gy >= (1 << 24) || g.gz >= (1 << 24)) return RC_ERR_TOO_LARGE;
    if (static_cast<double>(g.gx) * g.gy * g.gz >= 2147483648.0) return RC_ERR_TOO_LARGE;
    g.fgx = static_cast<float>(g.gx); g.fgy = static_cast<float>(g.gy); g.fgz = static_cast<float>(g.gz);
    g.inv_vs = host_reciprocal(voxel_size);
    const long long V = static_cast<long long>(g.gx) * g.gy * g.gz;
    if (chunks == 0 || V == 0) return RC_OK;
    if (N > 0 && (points == nullptr || features == nullptr)) return RC_ERR_NULL_POINTER;
    if (!rc::aligned_to(points, 4) || !rc::aligned_to(features, 16)) return RC_ERR_BAD_ALIGNMENT;
    ExchangeDest dest{};
    for (int d = 0; d < n_groups; ++d) {
        dest.ids[d] = static_cast<int*>(dest_ids[d]);
        dest.feats[d] = static_cast<float4*>(dest_features[d]);
        dest.runs[d] = static_cast<unsigned int*>(dest_runs[d]);
        if (dest.ids[d] == nullptr || dest.feats[d] == nullptr || dest.runs[d] == nullptr) return RC_ERR_NULL_POINTER;
        if (!rc::aligned_to(dest.ids[d], 128) || !rc::aligned_to(dest.feats[d], 128) || !rc::aligned_to(dest.runs[d], 4))
            return RC_ERR_BAD_ALIGNMENT;
    }
    const long long owner_span = ceil_div(V, n_groups);          // the ceil-div slabs the owners hold
    dest.groups = n_groups;
    dest.per_group = parts_per_group;
    dest.owner_span = static_cast<unsigned int>(owner_span);
    dest.inv_owner_span = 1.0f / static_cast<float>(owner_span);
    dest.block0 = first_block;
    dest.nblocks = pool_blocks;
    dest.bulk_store = rc::g_bucket_bulk_store.load(std::memory_order_relaxed) ? 1 : 0;
    RunRule rule;
    rule.P = n_groups * parts_per_group;
    rule.slab = static_cast<unsigned int>(ceil_div(owner_span, parts_per_group));
    rule.inv_slab = 1.0f / static_cast<float>(rule.slab);
    rule.blk = rc_voxel_bucket_block_records(parts_per_group);
    rc::DeviceScope scope(device);
    if (scope.status() != RC_OK) return scope.status();
    const int sms = rc::sm_count(device);
    const long long cap = static_cast<long long>(ctas_per_sm) * sms;
    const long long nb = chunks < cap ? chunks : cap;
    const int rc_smem = rc::ensure_dynamic_smem(reinterpret_cast<const void*>(voxel_bucket_kernel<true>), device, 2 * kBucketStageBytes);
    if (rc_smem != RC_OK) return rc_smem;
    voxel_bucket_kernel<true><<<static_cast<unsigned int>(nb), kThreads, 2 * kBucketStageBytes, static_cast<cudaStream_t>(stream)>>>(
        points, reinterpret_cast<const float4*>(features), N, g, rc::aligned_to(points, 16), rule, chunks, nullptr,
        nullptr, nullptr, dest, nullptr, 0);
    return rc::check_launch();
}

int rc_voxel_scatter_buckets(const void* const* pool_ids, const void* const* pool_features, const void* const* runs,
                             int32_t n_sources, int64_t blocks_per_source, int64_t table_row_blocks, int32_t parts_per_group,
                             float* grid, int32_t* counts, int64_t id_begin, int64_t id_end, uint32_t flags, int device,
                             void* stream) {
    if (n_sources < 0 || n_sources > kMeanRunsMaxParts || blocks_per_source < 0 || parts_per_group < 1 ||
        parts_per_group > kMeanRunsMaxParts || id_begin < 0 || id_end < id_begin)
        return RC_ERR_BAD_SHAPE;
    if (table_row_blocks == 0) table_row_blocks = blocks_per_source;
    if (table_row_blocks < blocks_per_source) return RC_ERR_BAD_SHAPE;
    if (id_end >= (1ll << 31)) return RC_ERR_TOO_LARGE;
    const long long nvox = id_end - id_begin;
    if (nvox > 0 && (grid == nullptr || counts == nullptr)) return RC_ERR_NULL_POINTER;
    const bool work = n_sources > 0 && blocks_per_source > 0 && nvox > 0;
    if (work && (pool_ids == nullptr || pool_features == nullptr || runs == nullptr)) return RC_ERR_NULL_POINTER;
    ScatterSources src{};
    src.n = n_sources;
    for (int i = 0; work && i < n_sources; ++i) {
        src.ids[i] = static_cast<const int*>(pool_ids[i]);
        src.feats[i] = static_cast<const float4*>(pool_features[i]);
        src.runs[i] = static_cast<const unsigned int*>(runs[i]);
        if (src.ids[i] == nullptr || src.feats[i] == nullptr || src.runs[i] == nullptr) return RC_ERR_NULL_POINTER;
        if (!rc::aligned_to(src.ids[i], 16) || !rc::aligned_to(src.feats[i], 16) || !rc::aligned_to(src.runs[i], 4))
            return RC_ERR_BAD_ALIGNMENT;
    }
    if (!rc::aligned_to(grid, 16) || !rc::aligned_to(counts, 4)) return RC_ERR_BAD_ALIGNMENT;
    rc::DeviceScope scope(device);
    if (scope.status() != RC_OK) return scope.status();
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if ((flags & RC_VOXEL_ZERO_INIT) && nvox > 0) {
        RC_CUDA_TRY(cudaMemsetAsync(grid, 0, static_cast<size_t>(nvox) * 16, st));
        RC_CUDA_TRY(cudaMemsetAsync(counts, 0, static_cast<size_t>(nvox) * 4, st));
    }
    if (work) {
        // the kernel indexes with the global id: hand it the address voxel 0 would have
        float* grid0 = reinterpret_cast<float*>(reinterpret_cast<uintptr_t>(grid) - static_cast<uintptr_t>(id_begin) * 16u);
        int* counts0 = reinterpret_cast<int*>(reinterpret_cast<uintptr_t>(counts) - static_cast<uintptr_t>(id_begin) * 4u);
        const int blk = rc_voxel_bucket_block_records(parts_per_group);
        const int sms = rc::sm_count(device);
        long long sb = ceil_div(blocks_per_source * n_sources, kThreads / 32);
        if (sb > 8ll * sms) sb = 8ll * sms;
        for (int k = 0; k < parts_per_group; ++k) {     // one launch per sub-range of the slab
            ScatterSources row = src;
            for (int i = 0; i < n_sources; ++i) row.runs[i] = src.runs[i] + static_cast<long long>(k) * table_row_blocks;
            bool launched = false;
            if (k > 0 && rc::g_scatter_overlap.load(std::memory_order_relaxed)) {
                cudaLaunchConfig_t cfg{};
                cfg.gridDim = dim3(static_cast<unsigned int>(sb));
                cfg.blockDim = dim3(kThreads);
                cfg.stream = st;
                cudaLaunchAttribute attr{};
                attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
                attr.val.programmaticStreamSerializationAllowed = 1;
                cfg.attrs = &attr;
                cfg.numAttrs = 1;
                launched = cudaLaunchKernelEx(&cfg, voxel_bucket_scatter_kernel, row, blocks_per_source, blk, grid0, counts0) == cudaSuccess;
                if (!launched) cudaGetLastError();
            }
            if (!launched)
                voxel_bucket_scatter_kernel<<<static_cast<unsigned int>(sb), kThreads, 0, st>>>(row, blocks_per_source, blk, grid0, counts0);
        }
    }
    const int rc_launch = rc::check_launch();
    if (rc_launch != RC_OK) return rc_launch;
    if (!(flags & RC_VOXEL_NO_NORMALIZE) && nvox > 0)
        return rc_voxel_normalize(grid, counts, 0, nvox, 4, device, stream);
    return RC_OK;
}

}  // extern "C"
