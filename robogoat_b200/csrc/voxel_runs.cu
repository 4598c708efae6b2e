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
//   scatter kernel  one launch per slab p: streams the runs of slab p (sequential reads: no random
//                   feature gather) into atomics that stay inside the slab, and - in the same
//                   warps, between runs - clears slab p+1 and normalises slab p-1
//                   (robocache/csrc/cuda/voxelize_kernel.cu:145-163).  The scatter is bound by the rate
//                   at which L2 retires atomics and leaves DRAM idle; the clear and the normalise are
//                   pure DRAM traffic, so running them underneath costs little.
//
// The bucket kernel clears slab 0; a last launch normalises the last slab.  Kernel boundaries order
// clear -> scatter -> normalise of a slab; no kernel waits on another.
#include "voxel_common.cuh"

namespace rc {
namespace vox {

namespace {

constexpr int kRunPad = 8;                                  // records: 32 bytes of ids, 128 bytes of feature rows
constexpr int kRunChunk = kPointsPerBlock;                  // 1024 points per CTA step
constexpr int kRunBlockMax = kRunChunk + kRunPad * kMeanRunsMaxParts;

struct RunRule {
    int P;                  // slabs in use
    unsigned int slab;      // voxel ids per slab, a multiple of 256
    float inv_slab;
    int blk;                // records per chunk block: 1024 + 8 * P
};

// n / d for quotients below kMeanRunsMaxParts and n < 2^31: float estimate, one correction step either way
__device__ __forceinline__ int slab_of(int id, const RunRule& r) {
    int q = static_cast<int>(__uint2float_rz(static_cast<unsigned int>(id)) * r.inv_slab);
    const long long lo = static_cast<long long>(q) * r.slab;
    if (id < lo) --q;
    else if (id >= lo + r.slab) ++q;
    return q;
}

// Clears voxels [a, b) of an F = 4 grid and of its counter plane.  a is a multiple of 4, both bases are
// 16-byte aligned; `t` of `nt` cooperating threads.
__device__ __forceinline__ void clear_voxels(float4* __restrict__ grid4, int* __restrict__ counts, long long a,
                                             long long b, int t, int nt) {
    const float4 z4 = make_float4(0.f, 0.f, 0.f, 0.f);
    for (long long v = a + t; v < b; v += nt) __stcs(grid4 + v, z4);
    const long long b4 = a + ((b - a) & ~3ll);
    int4* c4 = reinterpret_cast<int4*>(counts + a);
    const long long n4 = (b4 - a) >> 2;
    for (long long i = t; i < n4; i += nt) __stcs(c4 + i, make_int4(0, 0, 0, 0));
    for (long long v = b4 + t; v < b; v += nt) counts[v] = 0;
}

// grid[v,:] *= 1.0f / counts[v] for the occupied voxels of [a, b); a is a multiple of 4, one warp
__device__ __forceinline__ void normalize_voxels(float4* __restrict__ grid4, const int* __restrict__ counts, long long a,
                                                 long long b, int lane) {
    for (long long s = a; s < b; s += 128) {
        const long long v = s + lane * 4;
        int c[4] = {0, 0, 0, 0};
        if (v + 3 < b) {
            const int4 q = *reinterpret_cast<const int4*>(counts + v);
            c[0] = q.x; c[1] = q.y; c[2] = q.z; c[3] = q.w;
        } else {
#pragma unroll
            for (int k = 0; k < 4; ++k)
                if (v + k < b) c[k] = counts[v + k];
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            if (c[k] > 0) {     // empty voxels stay exactly 0
                const float inv = __fdiv_rn(1.0f, static_cast<float>(c[k]));
                float4 x = grid4[v + k];
                x.x = __fmul_rn(x.x, inv); x.y = __fmul_rn(x.y, inv);
                x.z = __fmul_rn(x.z, inv); x.w = __fmul_rn(x.w, inv);
                grid4[v + k] = x;
            }
        }
    }
}

// runs[p * nchunks + c] = (first slot of slab p's run in chunk c's block) << 16 | records in the run
__global__ void __launch_bounds__(kThreads, 4)
voxel_bucket_kernel(const float* __restrict__ pts, const float4* __restrict__ feats, long long N, VoxelGeom g,
                    bool pts_aligned, RunRule rule, long long nchunks, unsigned int* __restrict__ runs,
                    int* __restrict__ pool_ids, float4* __restrict__ pool_feats, bool clear, float4* __restrict__ grid4,
                    int* __restrict__ counts, long long clear_end, long long clear_piece,
                    const int* __restrict__ gate, int gate_want) {
    __shared__ __align__(16) float s_xyz[kThreads / 32][kPointsPerWarp * 3];
    __shared__ __align__(16) int s_sid[kRunBlockMax];
    __shared__ __align__(16) float4 s_sf[kRunBlockMax];
    __shared__ int s_wcnt[kThreads / 32][kMeanRunsMaxParts];
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
        const long long cbase = chunk * kRunChunk;
        const long long base = cbase + warp * kPointsPerWarp;
        const bool full = base + kPointsPerWarp <= N;
        float4 f[kPointsPerLane];
#pragma unroll
        for (int i = 0; i < kPointsPerLane; ++i) {
            const long long pi = base + i * 32 + lane;
            f[i] = (full || pi < N) ? __ldcs(feats + pi) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
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
            part[i] = (id[i] < 0) ? -1 : slab_of(id[i], rule);
        }
        // rank of every point among the warp's points of the same slab: intersect the ballots of the slab's bits
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
            rank[i] = 0;
            if (part[i] >= 0) rank[i] = wcnt[part[i]] + __popc(same & lt_mask);
            __syncwarp();
            if (part[i] >= 0 && (same & lt_mask) == 0u) wcnt[part[i]] += __popc(same);
            __syncwarp();
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
        for (int off = 1; off < 32; off <<= 1) {
            const int a = __shfl_up_sync(0xffffffffu, inc, off);
            if (lane >= off) inc += a;
        }
        const int total = __shfl_sync(0xffffffffu, inc, 31);
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
        if (warp == 0 && lane < P) {
            for (int j = start + tot; j < start + padded; ++j) s_sid[j] = -1;
            runs[static_cast<long long>(lane) * nchunks + chunk] = (static_cast<unsigned int>(start) << 16) | static_cast<unsigned int>(tot);
        }
        __syncthreads();
        if (lane < kMeanRunsMaxParts) wcnt[lane] = 0;     // own row, for the next chunk; every warp has read it
        {
            const long long o = chunk * rule.blk;
            int4* dst_i = reinterpret_cast<int4*>(pool_ids + o);
            const int4* src_i = reinterpret_cast<const int4*>(s_sid);
            for (int j = threadIdx.x; j < (total >> 2); j += kThreads) __stcs(dst_i + j, src_i[j]);
            float4* dst_f = pool_feats + o;
            for (int j = threadIdx.x; j < total; j += kThreads) __stcs(dst_f + j, s_sf[j]);
        }
        if (clear) {
            const long long a = chunk * clear_piece;
            const long long b = (a + clear_piece < clear_end) ? a + clear_piece : clear_end;
            if (a < b) clear_voxels(grid4, counts, a, b, threadIdx.x, kThreads);
        }
    }
}

// One slab's phase.  Warp w takes steps w, w + warps, ... of `iters`; step i accumulates the run of chunk i
// (i < nchunks), clears piece i of the next slab and normalises piece i of the previous one.
__global__ void __launch_bounds__(kThreads)
voxel_run_scatter_kernel(const unsigned int* __restrict__ runs_p, const int* __restrict__ pool_ids,
                         const float4* __restrict__ pool_feats, long long nchunks, int blk, float* __restrict__ grid,
                         int* __restrict__ counts, long long iters, long long clear_begin, long long clear_end,
                         long long clear_piece, long long norm_begin, long long norm_end, long long norm_piece,
                         const int* __restrict__ gate, int gate_want) {
    if (gate != nullptr && *gate != gate_want) return;
    const int lane = threadIdx.x & 31;
    const long long warps_total = static_cast<long long>(gridDim.x) * (kThreads / 32);
    float4* grid4 = reinterpret_cast<float4*>(grid);
    for (long long it = static_cast<long long>(blockIdx.x) * (kThreads / 32) + (threadIdx.x >> 5); it < iters; it += warps_total) {
        if (it < nchunks) {
            const unsigned int desc = __ldg(runs_p + it);
            const int n = static_cast<int>(desc & 0xffffu);
            const long long off = it * blk + (desc >> 16);
            for (int j0 = 0; j0 < n; j0 += kPointsPerWarp) {
                int id[kPointsPerLane];
                float4 f[kPointsPerLane];
#pragma unroll
                for (int i = 0; i < kPointsPerLane; ++i) {
                    const int j = j0 + i * 32 + lane;
                    id[i] = (j < n) ? __ldcs(pool_ids + off + j) : -1;
                    if (j < n) f[i] = __ldcs(pool_feats + off + j);
                }
#pragma unroll
                for (int i = 0; i < kPointsPerLane; ++i) {
                    if (id[i] >= 0) {
                        red_add_v4(grid + static_cast<long long>(id[i]) * 4, f[i]);
                        atomicAdd(counts + id[i], 1);
                    }
                }
            }
        }
        if (clear_piece > 0) {
            const long long a = clear_begin + it * clear_piece;
            const long long b = (a + clear_piece < clear_end) ? a + clear_piece : clear_end;
            if (a < b) clear_voxels(grid4, counts, a, b, lane, 32);
        }
        if (norm_piece > 0) {
            const long long a = norm_begin + it * norm_piece;
            const long long b = (a + norm_piece < norm_end) ? a + norm_piece : norm_end;
            if (a < b) normalize_voxels(grid4, counts, a, b, lane);
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
                     const VoxelGeom& g, long long V, int parts, bool clear, bool normalize, void* scratch,
                     const int* gate, int gate_want, int device, cudaStream_t st) {
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
    float4* grid4 = reinterpret_cast<float4*>(grid);

    const long long slab0_end = l.slab < V ? l.slab : V;
    long long nb = l.nchunks < 8ll * sms ? l.nchunks : 8ll * sms;
    voxel_bucket_kernel<<<static_cast<unsigned int>(nb), kThreads, 0, st>>>(
        points, reinterpret_cast<const float4*>(features), N, g, rc::aligned_to(points, 16), rule, l.nchunks, runs, pool_ids,
        pool_feats, clear, grid4, counts, slab0_end, round_up(ceil_div(slab0_end, l.nchunks), 256), gate, gate_want);

    // per-slab phases; the clear and normalise pieces are spread over at least one step per resident warp
    const long long min_iters = 8ll * sms * (kThreads / 32);
    const long long iters = l.nchunks > min_iters ? l.nchunks : min_iters;
    long long sb = ceil_div(iters, kThreads / 32);
    if (sb > 8ll * sms) sb = 8ll * sms;
    for (int p = 0; p <= l.P; ++p) {
        const bool scatter = p < l.P;
        const long long cb = static_cast<long long>(p + 1) * l.slab;           // slab p + 1
        const long long ce = cb + l.slab < V ? cb + l.slab : V;
        const bool do_clear = clear && scatter && cb < V;
        const long long nbeg = static_cast<long long>(p - 1) * l.slab;        // slab p - 1
        const long long nend = nbeg + l.slab < V ? nbeg + l.slab : V;
        const bool do_norm = normalize && p > 0;
        if (!scatter && !do_norm) break;
        voxel_run_scatter_kernel<<<static_cast<unsigned int>(sb), kThreads, 0, st>>>(
            runs + static_cast<long long>(scatter ? p : 0) * l.nchunks, pool_ids, pool_feats, scatter ? l.nchunks : 0, l.blk, grid,
            counts, iters, cb, ce, do_clear ? round_up(ceil_div(ce - cb, iters), 256) : 0, nbeg, nend,
            do_norm ? round_up(ceil_div(nend - nbeg, iters), 256) : 0, gate, gate_want);
    }
    return rc::check_launch();
}

}  // namespace vox
}  // namespace rc
