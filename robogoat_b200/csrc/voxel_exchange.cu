// Multi-GPU point exchange for voxelisation: instead of reducing dense partial grids, every rank
// buckets its points by the rank that owns their voxel (and by L2-sized sub-range of that rank's
// slab), the buckets travel to their owners - written by the move pass straight into the owners'
// memory, or by an all-to-all of the caller - and each owner accumulates the runs it received.
// No counterpart in the reference, whose multi-GPU test all-reduces dense grids
// (robocache/tests/test_multi_gpu.py:76).
#include "voxel_common.cuh"

#include <atomic>

namespace {

using namespace rc::vox;

// ---------------------------------------------------------------- partition by owning part (point exchange)
//
// A stable counting partition in three launches.  Every CTA owns a contiguous run of 1024-point
// chunks.  Launch 1 (MOVE = false) counts the in-grid points per CTA and part; launch 2 turns each
// part's column of that table into exclusive prefixes over the CTAs (one CTA per part); launch 3
// (MOVE = true) walks the same chunks again - the count pass leaves every point's voxel id in the
// scratch, so the coordinates are not read twice -, sorts each chunk by part in shared memory and writes
// the sorted chunk out, so that every part receives runs of consecutive records.  Ranks inside a
// warp come from ballots over the bits of the part number and warps are prefixed in order, so input
// order is kept inside a part and the result does not depend on scheduling.  For destinations on
// other GPUs the write-out is line-aligned (ALIGNED = true): every warp store covers one
// 32-record-aligned group of a destination, and records that do not fill a group yet wait in
// shared memory for the CTA's next chunk; the bytes that end up in the destinations are the same.
//
// Parts are two-level: n_groups owners (ranks) with ceil(V / n_groups) voxel ids each, every owner's
// range cut into parts_per_group sub-ranges of ceil(range / parts_per_group) ids; part = group *
// parts_per_group + sub.  Sub-ranges let the owner accumulate one L2-sized piece of its slab at a time.
constexpr int kMaxParts = 64;
constexpr int kChunk = kPointsPerBlock;   // 1024 points: one 128-point tile per warp

struct PartRule {
    unsigned int slab, sub;       // ids per group, ids per part inside a group
    float inv_slab, inv_sub;
    int per_group, P;
};

struct PartDest {                 // where the points of each part go (move pass)
    int* ids[kMaxParts];
    float* feats[kMaxParts];
    long long start[kMaxParts];   // first slot of this call's points in that buffer
};

// n / d and n % d for quotients up to a few hundred and n < 2^31: float estimate of the quotient, then
// one correction step either way on the 32-bit remainder
__device__ __forceinline__ unsigned int small_divmod(unsigned int n, unsigned int d, float inv, unsigned int* rem) {
    unsigned int q = static_cast<unsigned int>(__uint2float_rz(n) * inv);
    int r = static_cast<int>(n - q * d);
    if (r < 0) { --q; r += static_cast<int>(d); }
    else if (r >= static_cast<int>(d)) { ++q; r -= static_cast<int>(d); }
    *rem = static_cast<unsigned int>(r);
    return q;
}
__device__ __forceinline__ int part_of(int id, const PartRule& r) {
    unsigned int rem, rem2;
    const unsigned int grp = small_divmod(static_cast<unsigned int>(id), r.slab, r.inv_slab, &rem);
    const unsigned int k = small_divmod(rem, r.sub, r.inv_sub, &rem2);
    return static_cast<int>(grp) * r.per_group + static_cast<int>(k);
}

template <bool MOVE, bool ALIGNED>
__global__ void __launch_bounds__(kThreads, ALIGNED ? 4 : 5)
voxel_part_kernel(const float* __restrict__ pts, const float* __restrict__ feats, long long N, int F, VoxelGeom g,
                  bool pts_aligned, bool vec4, PartRule rule, long long chunks_per_cta, int* __restrict__ table,
                  int* __restrict__ ids_tmp, const long long* __restrict__ part_counts,
                  const __grid_constant__ PartDest dest) {
    __shared__ __align__(16) float s_xyz[MOVE ? 1 : kThreads / 32][MOVE ? 4 : kPointsPerWarp * 3];
    // count pass: per-warp totals.  move pass: this chunk's per-warp counts (every warp derives the
    // layout of the sorted chunk from them by itself)
    __shared__ int s_wcnt[kThreads / 32][kMaxParts];
    __shared__ long long s_cur[MOVE ? kMaxParts : 1];        // next slot of each part in its destination
    __shared__ int* s_adj_ids[MOVE ? kMaxParts : 1];         // destination of sorted slot j of part p is s_adj_*[p] + j
    __shared__ float* s_adj_feats[MOVE ? kMaxParts : 1];
    __shared__ int s_total;
    __shared__ int s_sid[MOVE ? kChunk : 1];                 // the chunk's voxel ids, sorted by part
    __shared__ unsigned short s_meta[MOVE ? kChunk : 1];     // (index in chunk << 6) | part
    // ALIGNED: every warp store covers one 32-slot-aligned group of a destination (a full 128-byte line of ids,
    // four full lines of feature rows) - what stores to a peer GPU need to run at link rate.  The records of a
    // part that do not fill a group yet wait here, as (voxel id, point index), for the next chunk.
    __shared__ int s_cid[ALIGNED ? kMaxParts : 1][ALIGNED ? 32 : 1];
    __shared__ int s_cpt[ALIGNED ? kMaxParts : 1][ALIGNED ? 32 : 1];
    __shared__ int s_cc[ALIGNED ? kMaxParts : 1];            // waiting records per part
    __shared__ int s_w[ALIGNED ? kMaxParts : 1];             // records of the part written with this chunk
    __shared__ int s_lst[ALIGNED ? kMaxParts : 1];           // start of the part's run in the sorted chunk
    __shared__ int s_tot[ALIGNED ? kMaxParts : 1];           // length of that run
    __shared__ int s_gstart[ALIGNED ? kMaxParts + 1 : 1];    // prefix of the parts' group counts
    __shared__ long long s_D[ALIGNED ? kMaxParts : 1];       // destination slot of the part's first unwritten record
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const unsigned int lt_mask = (1u << lane) - 1u;
    const int P = rule.P;
    const int nbits = 32 - __clz(P - 1 > 0 ? P - 1 : 1);                 // bits that tell the parts apart
    int* wcnt = s_wcnt[warp];
    for (int p = lane; p < P; p += 32) wcnt[p] = 0;
    if (MOVE) {
        for (int p = threadIdx.x; p < P; p += kThreads) {
            long long start;
            if (part_counts != nullptr) {          // local destination: parts packed back to back
                start = 0;
                for (int q = 0; q < p; ++q) start += part_counts[q];
            } else {
                start = dest.start[p];
            }
            s_cur[p] = start + table[static_cast<long long>(blockIdx.x) * P + p];
            if (ALIGNED) s_cc[p] = 0;
        }
    }
    __syncthreads();
    // N < 2^31 (checked by the host): point and chunk indices are 32-bit
    const int n_pts = static_cast<int>(N);
    const int nchunks = (n_pts + kChunk - 1) / kChunk;                  // n_pts + 1023 cannot overflow: N <= 2^31 - 1024 is enforced
    const int per_cta = static_cast<int>(chunks_per_cta);
    const int c0 = (static_cast<long long>(blockIdx.x) * per_cta < nchunks) ? static_cast<int>(blockIdx.x) * per_cta : nchunks;
    const int c1 = (nchunks - c0 > per_cta) ? c0 + per_cta : nchunks;
    const int toff = warp * kPointsPerWarp + lane;                      // this lane's first point inside a chunk
    float4 ahead[3];
    int ids_ahead[kPointsPerLane];
    if (c0 < c1) {
        const int tbase = c0 * kChunk + warp * kPointsPerWarp;
        if (MOVE) {
#pragma unroll
            for (int i = 0; i < kPointsPerLane; ++i) {
                const int pi = c0 * kChunk + toff + i * 32;
                ids_ahead[i] = (pi < n_pts) ? __ldcs(ids_tmp + pi) : -1;
            }
        } else if (pts_aligned && tbase + kPointsPerWarp <= n_pts) {
            tile_issue(pts, tbase, lane, ahead);
        }
    }
    for (int chunk = c0; chunk < c1; ++chunk) {
        const int cbase = chunk * kChunk;
        const int base = cbase + warp * kPointsPerWarp;
        const bool full = cbase + kChunk <= n_pts;                      // uniform: no per-point bound checks in full chunks
        const bool next_full = chunk + 1 < c1 && cbase + 2 * kChunk <= n_pts;
        int id[kPointsPerLane], part[kPointsPerLane], rank[kPointsPerLane];
        if (MOVE) {
            // the voxel ids were left behind by the count pass; fetch the next chunk's while this one is sorted
#pragma unroll
            for (int i = 0; i < kPointsPerLane; ++i) id[i] = ids_ahead[i];
            if (next_full) {
#pragma unroll
                for (int i = 0; i < kPointsPerLane; ++i) ids_ahead[i] = __ldcs(ids_tmp + cbase + kChunk + toff + i * 32);
            } else {
#pragma unroll
                for (int i = 0; i < kPointsPerLane; ++i) {
                    const int pn = cbase + kChunk + toff + i * 32;
                    ids_ahead[i] = (chunk + 1 < c1 && pn < n_pts) ? __ldcs(ids_tmp + pn) : -1;
                }
            }
        } else {
            float x[kPointsPerLane], y[kPointsPerLane], z[kPointsPerLane];
            if (pts_aligned && (full || base + kPointsPerWarp <= n_pts)) {
                float4 now[3] = {ahead[0], ahead[1], ahead[2]};
                const int nbase = base + kChunk;
                if (next_full || (chunk + 1 < c1 && nbase + kPointsPerWarp <= n_pts)) tile_issue(pts, nbase, lane, ahead);
                tile_unpack(now, s_xyz[warp], lane, x, y, z);
            } else {
                tile_load_slow(pts, base, N, lane, x, y, z);
            }
            if (full) {
#pragma unroll
                for (int i = 0; i < kPointsPerLane; ++i) {
                    id[i] = voxel_id32(x[i], y[i], z[i], g);
                    __stcs(ids_tmp + cbase + toff + i * 32, id[i]);
                }
            } else {
#pragma unroll
                for (int i = 0; i < kPointsPerLane; ++i) {
                    const int pi = cbase + toff + i * 32;
                    id[i] = (pi < n_pts) ? voxel_id32(x[i], y[i], z[i], g) : -1;
                    if (pi < n_pts) __stcs(ids_tmp + pi, id[i]);
                }
            }
        }
#pragma unroll
        for (int i = 0; i < kPointsPerLane; ++i) part[i] = (id[i] < 0) ? -1 : part_of(id[i], rule);
        if (!MOVE) {
            // counting needs no order: shared-memory atomics on the warp's own row
#pragma unroll
            for (int i = 0; i < kPointsPerLane; ++i)
                if (part[i] >= 0) atomicAdd(&wcnt[part[i]], 1);
            continue;
        }
#pragma unroll
        for (int i = 0; i < kPointsPerLane; ++i) {
            // lanes holding the same part: intersect the ballots of the part's six bits (cheaper than
            // __match_any_sync when a row holds many different parts)
            unsigned int same = __ballot_sync(0xffffffffu, part[i] >= 0);
#pragma unroll
            for (int bit = 0; bit < 6; ++bit) {
                if (bit < nbits) {                                       // uniform
                    const bool on = (part[i] >> bit) & 1;
                    const unsigned int b = __ballot_sync(0xffffffffu, on);
                    same &= on ? b : ~b;
                }
            }
            rank[i] = 0;
            if (part[i] >= 0) rank[i] = wcnt[part[i]] + __popc(same & lt_mask);
            __syncwarp();
            if (part[i] >= 0 && (same & lt_mask) == 0u) wcnt[part[i]] += __popc(same);   // lowest lane of the group
            __syncwarp();
        }
        __syncthreads();   // every warp's counts are in; the previous chunk's sorted arrays are no longer read
        // Every warp works out the layout of the sorted chunk by itself (no second barrier, no serial phase):
        // lane p, and p + 32 when there are more than 32 parts, sums part p over the warps, the totals are
        // prefixed over the parts with shuffles, and the lane keeps the first sorted slot of this warp's
        // points of its part(s) in registers.
        const bool wide = P > 32;                                   // uniform: the upper half is skipped for <= 32 parts
        int tot[2] = {0, 0}, mine[2] = {0, 0};
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int p = lane + 32 * h;
            if ((h == 0 || wide) && p < P) {
#pragma unroll
                for (int w = 0; w < kThreads / 32; ++w) {
                    const int t = s_wcnt[w][p];
                    if (w < warp) mine[h] += t;
                    tot[h] += t;
                }
            }
        }
        int inc0 = tot[0], inc1 = tot[1];
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const int a = __shfl_up_sync(0xffffffffu, inc0, off);
            if (lane >= off) inc0 += a;
        }
        if (wide) {
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const int b = __shfl_up_sync(0xffffffffu, inc1, off);
                if (lane >= off) inc1 += b;
            }
        }
        const int sum0 = __shfl_sync(0xffffffffu, inc0, 31);
        const int lstart[2] = {inc0 - tot[0], sum0 + inc1 - tot[1]};
        const int first0 = lstart[0] + mine[0], first1 = lstart[1] + mine[1];
        if (warp == 0) {   // destinations of the sorted slots, advanced by this chunk
            if (lane == 31) s_total = sum0 + inc1;
            if (!ALIGNED) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int p = lane + 32 * h;
                    if (p < P) {
                        const long long first = s_cur[p] - lstart[h];
                        s_adj_ids[p] = dest.ids[p] + first;
                        s_adj_feats[p] = (dest.feats[p] != nullptr) ? dest.feats[p] + first * F : nullptr;
                        s_cur[p] += tot[h];
                    }
                }
            } else {
                // per part: the stream to write is the waiting records followed by this chunk's run; everything
                // up to the last full group goes out now (all of it with the CTA's last chunk)
                const bool last = chunk == c1 - 1;
                int groups[2] = {0, 0};
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int p = lane + 32 * h;
                    if (p < P) {
                        const long long D = s_cur[p];
                        const int hh = static_cast<int>(D & 31);
                        const int n = s_cc[p] + tot[h];
                        int w = last ? n : (((hh + n) & ~31) - hh);
                        if (w < 0) w = 0;
                        groups[h] = (w > 0) ? ((hh + w + 31) >> 5) : 0;
                        s_w[p] = w; s_lst[p] = lstart[h]; s_tot[p] = tot[h]; s_D[p] = D;
                        s_cur[p] = D + w;
                    }
                }
                int g0 = groups[0], g1 = groups[1];
#pragma unroll
                for (int off = 1; off < 32; off <<= 1) {
                    const int a = __shfl_up_sync(0xffffffffu, g0, off);
                    const int b = __shfl_up_sync(0xffffffffu, g1, off);
                    if (lane >= off) { g0 += a; g1 += b; }
                }
                const int gsum0 = __shfl_sync(0xffffffffu, g0, 31);
                if (lane < P) s_gstart[lane + 1] = g0;                       // inclusive prefix = start of the next part
                if (lane + 32 < P) s_gstart[lane + 33] = gsum0 + g1;
                if (lane == 0) s_gstart[0] = 0;
            }
        }
#pragma unroll
        for (int i = 0; i < kPointsPerLane; ++i) {
            const int src_lane = part[i] & 31;                      // all lanes take part in the shuffles
            const int f0 = __shfl_sync(0xffffffffu, first0, src_lane);
            const int f1 = wide ? __shfl_sync(0xffffffffu, first1, src_lane) : 0;
            if (part[i] >= 0) {
                const int slot = ((part[i] < 32) ? f0 : f1) + rank[i];
                s_sid[slot] = id[i];
                s_meta[slot] = static_cast<unsigned short>(((warp * kPointsPerWarp + i * 32 + lane) << 6) | part[i]);
            }
        }
        __syncthreads();
        for (int p = lane; p < P; p += 32) wcnt[p] = 0;      // own row, for the next chunk; every warp has read it
        if (ALIGNED) {
            const int G = s_gstart[P];
            constexpr int kUnroll = 4;                       // groups per warp in flight: their feature loads overlap
            for (int g0 = warp; g0 < G; g0 += kUnroll * (kThreads / 32)) {
                int vid[kUnroll], pidx[kUnroll], pp[kUnroll];
                long long slot[kUnroll];
#pragma unroll
                for (int u = 0; u < kUnroll; ++u) {
                    const int g = g0 + u * (kThreads / 32);
                    pp[u] = -1;
                    if (g < G) {                             // uniform
                        // the part whose groups contain g: as many parts end at or before g
                        int p = __popc(__ballot_sync(0xffffffffu, lane < P && s_gstart[lane + 1] <= g));
                        if (P > 32) p += __popc(__ballot_sync(0xffffffffu, lane + 32 < P && s_gstart[lane + 33] <= g));
                        const long long D = s_D[p];
                        const int r = (g - s_gstart[p]) * 32 + lane - static_cast<int>(D & 31);   // record of the part's stream
                        if (r >= 0 && r < s_w[p]) {
                            const int c = s_cc[p];
                            if (r < c) {
                                vid[u] = s_cid[p][r];
                                pidx[u] = s_cpt[p][r];
                            } else {
                                const int j = s_lst[p] + r - c;
                                vid[u] = s_sid[j];
                                pidx[u] = cbase + (s_meta[j] >> 6);
                            }
                            slot[u] = D + r;
                            pp[u] = p;
                        }
                    }
                }
                if (vec4) {
                    float4 f4[kUnroll];
#pragma unroll
                    for (int u = 0; u < kUnroll; ++u)
                        if (pp[u] >= 0) f4[u] = __ldcs(reinterpret_cast<const float4*>(feats) + pidx[u]);
#pragma unroll
                    for (int u = 0; u < kUnroll; ++u) {
                        if (pp[u] >= 0) {
                            dest.ids[pp[u]][slot[u]] = vid[u];
                            reinterpret_cast<float4*>(dest.feats[pp[u]])[slot[u]] = f4[u];
                        }
                    }
                } else {
#pragma unroll
                    for (int u = 0; u < kUnroll; ++u) {
                        if (pp[u] >= 0) {
                            dest.ids[pp[u]][slot[u]] = vid[u];
                            float* fo = dest.feats[pp[u]];
                            if (fo != nullptr) {
                                const float* fi = feats + static_cast<long long>(pidx[u]) * F;
                                for (int ch = 0; ch < F; ++ch) fo[slot[u] * F + ch] = __ldg(fi + ch);
                            }
                        }
                    }
                }
            }
            __syncthreads();   // the waiting records have been read; now replace them
            for (int sl = threadIdx.x; sl < P * 32; sl += kThreads) {
                const int p = sl >> 5, i = sl & 31;           // one warp per part: its 32 waiting slots
                const int c = s_cc[p], w = s_w[p], n = c + s_tot[p];
                const int r = i + w;
                if (r >= (w > c ? w : c) && r < n) {          // records of this chunk's run that stay behind
                    const int j = s_lst[p] + r - c;
                    s_cid[p][i] = s_sid[j];
                    s_cpt[p][i] = cbase + (s_meta[j] >> 6);
                }
                __syncwarp();
                if (i == 0) s_cc[p] = n - w;
            }
        } else {
            const int n = s_total;
            if (vec4) {
                float4 f4[kPointsPerLane];
                int meta[kPointsPerLane];
    #pragma unroll
                for (int m = 0; m < kPointsPerLane; ++m) {
                    const int j = threadIdx.x + m * kThreads;
                    meta[m] = (j < n) ? s_meta[j] : -1;
                    if (j < n) f4[m] = __ldcs(reinterpret_cast<const float4*>(feats) + (cbase + (meta[m] >> 6)));
                }
    #pragma unroll
                for (int m = 0; m < kPointsPerLane; ++m) {
                    const int j = threadIdx.x + m * kThreads;
                    if (meta[m] >= 0) {
                        const int p = meta[m] & 63;
                        s_adj_ids[p][j] = s_sid[j];
                        reinterpret_cast<float4*>(s_adj_feats[p])[j] = f4[m];
                    }
                }
            } else {
                for (int j = threadIdx.x; j < n; j += kThreads) {
                    const int meta = s_meta[j];
                    const int p = meta & 63;
                    s_adj_ids[p][j] = s_sid[j];
                    float* fo = s_adj_feats[p];
                    if (fo != nullptr) {
                        const float* fi = feats + static_cast<long long>(cbase + (meta >> 6)) * F;
                        for (int c = 0; c < F; ++c) fo[static_cast<long long>(j) * F + c] = __ldg(fi + c);
                    }
                }
            }
        }
        // no barrier here: the next chunk's first barrier comes before anything above is overwritten
    }
    if (!MOVE) {
        __syncthreads();
        for (int p = threadIdx.x; p < P; p += kThreads) {
            int c = 0;
            for (int w = 0; w < kThreads / 32; ++w) c += s_wcnt[w][p];
            table[static_cast<long long>(blockIdx.x) * P + p] = c;
        }
    }
}

// CTA p: exclusive prefix over the CTAs of column p of the table, total into part_counts[p]
__global__ void __launch_bounds__(1024)
voxel_part_scan_kernel(int* __restrict__ table, long long W, int P, long long* __restrict__ part_counts) {
    __shared__ long long s_sum[1024];
    const int p = blockIdx.x;
    const long long per = (W + 1023) / 1024;
    const long long a = threadIdx.x * per;
    const long long b = (a + per < W) ? a + per : W;
    long long mine = 0;
    for (long long w = a; w < b; ++w) mine += table[w * P + p];
    s_sum[threadIdx.x] = mine;
    __syncthreads();
    for (int off = 1; off < 1024; off <<= 1) {   // inclusive scan of the per-thread sums
        const long long add = (threadIdx.x >= off) ? s_sum[threadIdx.x - off] : 0;
        __syncthreads();
        s_sum[threadIdx.x] += add;
        __syncthreads();
    }
    long long run = s_sum[threadIdx.x] - mine;
    for (long long w = a; w < b; ++w) {
        const int c = table[w * P + p];
        table[w * P + p] = static_cast<int>(run);
        run += c;
    }
    if (threadIdx.x == 1023) part_counts[p] = s_sum[1023];
}

// CTAs that share the chunks of a cloud of N points
void partition_plan(long long N, int device, long long* blocks, long long* chunks_per_cta) {
    const long long nchunks = (N + kChunk - 1) / kChunk;
    long long nb = nchunks;
    const long long cap = 16ll * rc::sm_count(device);
    if (nb > cap) nb = cap;
    if (nb < 1) nb = 1;
    *chunks_per_cta = (nchunks + nb - 1) / nb;
    *blocks = nb;
}

// scratch layout of the partition: per-block offsets [blocks][P] int32, then the voxel id of every point
uint64_t partition_table_bytes(long long blocks, int P) {
    return (static_cast<uint64_t>(blocks) * static_cast<uint64_t>(P) * 4u + 15u) & ~static_cast<uint64_t>(15);
}

int partition_geometry(const float grid_min_host[3], float voxel_size, const int32_t grid_size_host[3], int32_t n_groups,
                       int32_t parts_per_group, VoxelGeom* g, PartRule* rule, long long* V_out) {
    if (grid_min_host == nullptr || grid_size_host == nullptr) return RC_ERR_NULL_POINTER;
    if (n_groups < 1 || parts_per_group < 1) return RC_ERR_BAD_SHAPE;
    if (static_cast<long long>(n_groups) * parts_per_group > kMaxParts) return RC_ERR_TOO_LARGE;
    if (!(voxel_size > 0.0f) || !(voxel_size <= 3.0e38f)) return RC_ERR_BAD_VALUE;
    g->minx = grid_min_host[0]; g->miny = grid_min_host[1]; g->minz = grid_min_host[2];
    g->vs = voxel_size;
    g->gx = grid_size_host[0]; g->gy = grid_size_host[1]; g->gz = grid_size_host[2];
    if (g->gx < 0 || g->gy < 0 || g->gz < 0) return RC_ERR_BAD_SHAPE;
    if (g->gx >= (1 << 24) || g->gy >= (1 << 24) || g->gz >= (1 << 24)) return RC_ERR_TOO_LARGE;
    if (static_cast<double>(g->gx) * g->gy * g->gz >= 2147483648.0) return RC_ERR_TOO_LARGE;
    g->fgx = static_cast<float>(g->gx); g->fgy = static_cast<float>(g->gy); g->fgz = static_cast<float>(g->gz);
    g->inv_vs = host_reciprocal(voxel_size);
    const long long V = static_cast<long long>(g->gx) * g->gy * g->gz;
    *V_out = V;
    const long long slab = (V + n_groups - 1) / n_groups;
    const long long sub = (slab + parts_per_group - 1) / parts_per_group;
    rule->slab = static_cast<unsigned int>(slab > 0 ? slab : 1);
    rule->sub = static_cast<unsigned int>(sub > 0 ? sub : 1);
    rule->inv_slab = 1.0f / static_cast<float>(rule->slab);
    rule->inv_sub = 1.0f / static_cast<float>(rule->sub);
    rule->per_group = parts_per_group;
    rule->P = n_groups * parts_per_group;
    return RC_OK;
}

// ---------------------------------------------------------------- scatter of pre-sorted runs
//
// The owner's side of the point exchange.  What arrives is a list of runs, each holding the points
// of one sub-range of the slab; the runs of one sub-range are accumulated by one launch, so its
// atomics work on an L2-sized piece of the slab and the records stream in sequentially.
struct RunTable {
    long long begin[kMaxParts];
    long long count[kMaxParts];
    long long first_block[kMaxParts + 1];   // in blocks of kChunk points
    int n;
};

template <int MODE>
__global__ void __launch_bounds__(kThreads)
voxel_scatter_runs_kernel(const int* __restrict__ ids, const float* __restrict__ feats, void* __restrict__ grid_v,
                          int* __restrict__ counts, int F, bool vec4, const __grid_constant__ RunTable rt, int id_lo,
                          unsigned int span) {
    // the next pass depends on this one's order (L2 locality) only, not on its results: launched as a programmatic
    // dependent it may fill the SMs this pass's last CTAs leave idle
    grid_dependency_release();
    const long long total = rt.first_block[rt.n];
    for (long long b = blockIdx.x; b < total; b += gridDim.x) {
        int r = 0;
        while (r + 1 < rt.n && rt.first_block[r + 1] <= b) ++r;
        const long long off = (b - rt.first_block[r]) * kChunk;
        const long long cnt = rt.count[r];
        const long long p0 = rt.begin[r];
        int id[kPointsPerLane];
        float4 f4[kPointsPerLane];
#pragma unroll
        for (int m = 0; m < kPointsPerLane; ++m) {
            const long long j = off + m * kThreads + threadIdx.x;
            id[m] = (j < cnt) ? __ldcs(ids + p0 + j) : -1;
            if (MODE == kMean && vec4 && j < cnt) f4[m] = __ldcs(reinterpret_cast<const float4*>(feats) + p0 + j);
        }
#pragma unroll
        for (int m = 0; m < kPointsPerLane; ++m) {
            if (static_cast<unsigned int>(id[m] - id_lo) >= span) continue;   // also drops -1 and foreign ids
            if (MODE == kMean && vec4) {
                red_add_v4(static_cast<float*>(grid_v) + static_cast<long long>(id[m]) * 4, f4[m]);
                atomicAdd(counts + id[m], 1);
            } else {
                scatter_one<MODE>(id[m], p0 + off + m * kThreads + threadIdx.x, feats, grid_v, counts, F);
            }
        }
    }
}

template <int MODE>
void launch_scatter_runs(bool overlap_prev, unsigned int nb, cudaStream_t st, const int* ids, const float* feats, void* grid0,
                         int* counts0, int F, bool vec4, const RunTable& rt, int id_lo, unsigned int span) {
    if (overlap_prev && rc::g_scatter_overlap.load(std::memory_order_relaxed)) {
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(nb);
        cfg.blockDim = dim3(kThreads);
        cfg.stream = st;
        cudaLaunchAttribute attr{};
        attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr.val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        if (cudaLaunchKernelEx(&cfg, voxel_scatter_runs_kernel<MODE>, ids, feats, grid0, counts0, F, vec4, rt, id_lo, span) == cudaSuccess)
            return;
        cudaGetLastError();  // attribute refused: an ordinary launch
    }
    voxel_scatter_runs_kernel<MODE><<<nb, kThreads, 0, st>>>(ids, feats, grid0, counts0, F, vec4, rt, id_lo, span);
}

}  // namespace

extern "C" {

uint64_t rc_voxel_partition_scratch_bytes(int64_t N, int32_t n_parts, int device) {
    if (N <= 0 || n_parts < 1 || n_parts > kMaxParts) return 0;
    long long blocks = 0, per = 0;
    partition_plan(N, device, &blocks, &per);
    return partition_table_bytes(blocks, n_parts) + static_cast<uint64_t>(N) * 4u;
}

int rc_voxel_partition_count(const float* points, int64_t N, const float grid_min_host[3], float voxel_size,
                             const int32_t grid_size_host[3], int32_t n_groups, int32_t parts_per_group,
                             int64_t* part_counts, void* scratch, uint64_t scratch_bytes, int device, void* stream) {
    VoxelGeom g;
    PartRule rule;
    long long V = 0;
    const int rc_geom = partition_geometry(grid_min_host, voxel_size, grid_size_host, n_groups, parts_per_group, &g, &rule, &V);
    if (rc_geom != RC_OK) return rc_geom;
    if (part_counts == nullptr) return RC_ERR_NULL_POINTER;
    if (N < 0) return RC_ERR_BAD_SHAPE;
    if (N > (1ll << 31) - 4096) return RC_ERR_TOO_LARGE;   // 32-bit point indices with room for one chunk of look-ahead
    if (N > 0 && points == nullptr) return RC_ERR_NULL_POINTER;
    if (!rc::aligned_to(points, 4) || !rc::aligned_to(part_counts, 8)) return RC_ERR_BAD_ALIGNMENT;
    rc::DeviceScope scope(device);
    if (scope.status() != RC_OK) return scope.status();
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (N == 0 || V == 0) {
        RC_CUDA_TRY(cudaMemsetAsync(part_counts, 0, static_cast<size_t>(rule.P) * 8, st));
        return RC_OK;
    }
    long long blocks = 0, per = 0;
    partition_plan(N, device, &blocks, &per);
    if (scratch == nullptr) return RC_ERR_NULL_POINTER;
    if (!rc::aligned_to(scratch, 16)) return RC_ERR_BAD_ALIGNMENT;
    if (scratch_bytes < partition_table_bytes(blocks, rule.P) + static_cast<uint64_t>(N) * 4u) return RC_ERR_BAD_SHAPE;
    int* table = static_cast<int*>(scratch);
    int* ids_tmp = reinterpret_cast<int*>(static_cast<unsigned char*>(scratch) + partition_table_bytes(blocks, rule.P));
    PartDest none{};
    voxel_part_kernel<false, false><<<static_cast<unsigned int>(blocks), kThreads, 0, st>>>(
        points, nullptr, N, 0, g, rc::aligned_to(points, 16), false, rule, per, table, ids_tmp, nullptr, none);
    voxel_part_scan_kernel<<<rule.P, 1024, 0, st>>>(table, blocks, rule.P, reinterpret_cast<long long*>(part_counts));
    return rc::check_launch();
}

int rc_voxel_partition_move(const float* points, const float* features, int64_t N, int32_t F,
                            const float grid_min_host[3], float voxel_size, const int32_t grid_size_host[3],
                            int32_t n_groups, int32_t parts_per_group, void* const* dest_ids, void* const* dest_features,
                            const int64_t* dest_start, const int64_t* part_counts_device, uint32_t flags,
                            const void* scratch, uint64_t scratch_bytes, int device, void* stream) {
    VoxelGeom g;
    PartRule rule;
    long long V = 0;
    const int rc_geom = partition_geometry(grid_min_host, voxel_size, grid_size_host, n_groups, parts_per_group, &g, &rule, &V);
    if (rc_geom != RC_OK) return rc_geom;
    if (N < 0 || F < 0) return RC_ERR_BAD_SHAPE;
    if (N > (1ll << 31) - 4096) return RC_ERR_TOO_LARGE;   // 32-bit point indices with room for one chunk of look-ahead
    if (N == 0 || V == 0) return RC_OK;
    if (points == nullptr || dest_ids == nullptr || scratch == nullptr) return RC_ERR_NULL_POINTER;
    if (dest_start == nullptr && part_counts_device == nullptr) return RC_ERR_NULL_POINTER;
    const bool move_feats = features != nullptr && dest_features != nullptr && F > 0;
    PartDest dest{};
    bool all16 = rc::aligned_to(features, 16);
    for (int p = 0; p < rule.P; ++p) {
        dest.ids[p] = static_cast<int*>(dest_ids[p]);
        dest.feats[p] = move_feats ? static_cast<float*>(dest_features[p]) : nullptr;
        dest.start[p] = dest_start != nullptr ? dest_start[p] : 0;
        if (dest.ids[p] == nullptr || (move_feats && dest.feats[p] == nullptr)) return RC_ERR_NULL_POINTER;
        if (dest.start[p] < 0) return RC_ERR_BAD_SHAPE;
        if (!rc::aligned_to(dest.ids[p], 4) || !rc::aligned_to(dest.feats[p], 4)) return RC_ERR_BAD_ALIGNMENT;
        all16 = all16 && rc::aligned_to(dest.feats[p], 16);
    }
    if (!rc::aligned_to(points, 4) || !rc::aligned_to(features, 4) || !rc::aligned_to(scratch, 16)) return RC_ERR_BAD_ALIGNMENT;
    rc::DeviceScope scope(device);
    if (scope.status() != RC_OK) return scope.status();
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    long long blocks = 0, per = 0;
    partition_plan(N, device, &blocks, &per);
    if (scratch_bytes < partition_table_bytes(blocks, rule.P) + static_cast<uint64_t>(N) * 4u) return RC_ERR_BAD_SHAPE;
    const bool vec4 = move_feats && F == 4 && all16;
    // line-aligned warp stores pay off over NVLink; in local memory L2 merges partial lines anyway
    const int aligned_opt = rc::g_part_aligned_store.load(std::memory_order_relaxed);
    const bool line_aligned = aligned_opt == 2 || (aligned_opt == 1 && (flags & RC_PARTITION_REMOTE_DESTINATIONS) != 0);
    int* table = const_cast<int*>(static_cast<const int*>(scratch));
    int* ids_tmp = reinterpret_cast<int*>(const_cast<unsigned char*>(static_cast<const unsigned char*>(scratch)) +
                                          partition_table_bytes(blocks, rule.P));
    const unsigned int nb = static_cast<unsigned int>(blocks);
    const float* f_in = move_feats ? features : nullptr;
    const long long* pc_dev = reinterpret_cast<const long long*>(part_counts_device);
    if (line_aligned)
        voxel_part_kernel<true, true><<<nb, kThreads, 0, st>>>(points, f_in, N, F, g, rc::aligned_to(points, 16), vec4, rule, per,
                                                               table, ids_tmp, pc_dev, dest);
    else
        voxel_part_kernel<true, false><<<nb, kThreads, 0, st>>>(points, f_in, N, F, g, rc::aligned_to(points, 16), vec4, rule, per,
                                                                table, ids_tmp, pc_dev, dest);
    return rc::check_launch();
}

int rc_voxel_partition(const float* points, const float* features, int64_t N, int32_t F,
                       const float grid_min_host[3], float voxel_size, const int32_t grid_size_host[3],
                       int32_t n_groups, int32_t parts_per_group, int32_t* ids_out, float* features_out,
                       int64_t* part_counts, void* scratch, uint64_t scratch_bytes, int device, void* stream) {
    const int rc_count = rc_voxel_partition_count(points, N, grid_min_host, voxel_size, grid_size_host, n_groups,
                                                  parts_per_group, part_counts, scratch, scratch_bytes, device, stream);
    if (rc_count != RC_OK) return rc_count;
    if (N > 0 && ids_out == nullptr) return RC_ERR_NULL_POINTER;
    void* ids_of[kMaxParts];
    void* feats_of[kMaxParts];
    for (int p = 0; p < kMaxParts; ++p) { ids_of[p] = ids_out; feats_of[p] = features_out; }
    return rc_voxel_partition_move(points, features, N, F, grid_min_host, voxel_size, grid_size_host, n_groups,
                                   parts_per_group, ids_of, features_out != nullptr ? feats_of : nullptr, nullptr,
                                   part_counts, 0u, scratch, scratch_bytes, device, stream);
}

int rc_voxel_scatter_runs(const int32_t* ids, const float* features, void* grid, int32_t* counts, int32_t F,
                          int64_t id_begin, int64_t id_end, const int64_t* run_begin, const int64_t* run_count,
                          const int32_t* run_pass, int32_t n_runs, int32_t n_passes, int mode, uint32_t flags,
                          int device, void* stream) {
    if (mode != RC_VOXEL_COUNT && mode != RC_VOXEL_OCCUPANCY && mode != RC_VOXEL_MEAN) return RC_ERR_BAD_MODE;
    if (F < 0 || id_begin < 0 || id_end < id_begin || n_runs < 0 || n_passes < 0) return RC_ERR_BAD_SHAPE;
    if (id_end >= (1ll << 31)) return RC_ERR_TOO_LARGE;
    if (n_runs > 0 && (run_begin == nullptr || run_count == nullptr || run_pass == nullptr)) return RC_ERR_NULL_POINTER;
    const long long nvox = id_end - id_begin;
    const bool mean = (mode == RC_VOXEL_MEAN);
    long long total = 0;
    for (int r = 0; r < n_runs; ++r) {
        if (run_begin[r] < 0 || run_count[r] < 0 || run_pass[r] < 0 || run_pass[r] >= n_passes) return RC_ERR_BAD_SHAPE;
        total += run_count[r];
    }
    if (nvox > 0 && (!mean || F > 0) && grid == nullptr) return RC_ERR_NULL_POINTER;
    if (mean && nvox > 0 && counts == nullptr) return RC_ERR_NULL_POINTER;
    if (total > 0 && ids == nullptr) return RC_ERR_NULL_POINTER;
    if (mean && total > 0 && F > 0 && features == nullptr) return RC_ERR_BAD_MODE;
    if (!rc::aligned_to(ids, 4) || !rc::aligned_to(grid, 4) || !rc::aligned_to(counts, 4) || !rc::aligned_to(features, 4))
        return RC_ERR_BAD_ALIGNMENT;
    if (mean) {
        const bool a16 = rc::aligned_to(features, 16) && rc::aligned_to(grid, 16);
        const bool a8 = rc::aligned_to(features, 8) && rc::aligned_to(grid, 8);
        if ((F & 3) == 0 && !a16) return RC_ERR_BAD_ALIGNMENT;
        if ((F & 3) != 0 && (F & 1) == 0 && !a8) return RC_ERR_BAD_ALIGNMENT;
    }
    rc::DeviceScope scope(device);
    if (scope.status() != RC_OK) return scope.status();
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const long long cells = mean ? nvox * F : nvox;
    if (flags & RC_VOXEL_ZERO_INIT) {
        if (cells > 0) RC_CUDA_TRY(cudaMemsetAsync(grid, 0, static_cast<size_t>(cells) * 4, st));
        if (mean && nvox > 0) RC_CUDA_TRY(cudaMemsetAsync(counts, 0, static_cast<size_t>(nvox) * 4, st));
    }
    if (total > 0 && nvox > 0 && !(mean && F == 0)) {
        const uintptr_t cell = mean ? static_cast<uintptr_t>(F) * 4u : 4u;
        void* grid0 = reinterpret_cast<void*>(reinterpret_cast<uintptr_t>(grid) - static_cast<uintptr_t>(id_begin) * cell);
        int* counts0 = mean ? reinterpret_cast<int*>(reinterpret_cast<uintptr_t>(counts) - static_cast<uintptr_t>(id_begin) * 4u)
                            : nullptr;
        const bool vec4 = mean && F == 4;
        const long long cap = 16ll * rc::sm_count(device);
        int launches = 0;       // the first launch waits for whatever precedes it on the stream (the clear); later ones may overlap
        for (int ps = 0; ps < n_passes; ++ps) {
            RunTable rt{};
            auto flush = [&]() {
                if (rt.n == 0) return;
                const bool ov = launches++ > 0;
                long long nb = rt.first_block[rt.n];
                if (nb > cap) nb = cap;
                const unsigned int blocks = static_cast<unsigned int>(nb);
                const int lo = static_cast<int>(id_begin);
                const unsigned int span = static_cast<unsigned int>(nvox);
                if (mode == RC_VOXEL_MEAN) launch_scatter_runs<kMean>(ov, blocks, st, ids, features, grid0, counts0, F, vec4, rt, lo, span);
                else if (mode == RC_VOXEL_COUNT) launch_scatter_runs<kCount>(ov, blocks, st, ids, features, grid0, counts0, F, false, rt, lo, span);
                else launch_scatter_runs<kOccupancy>(ov, blocks, st, ids, features, grid0, counts0, F, false, rt, lo, span);
                rt = RunTable{};
            };
            for (int r = 0; r < n_runs; ++r) {
                if (run_pass[r] != ps || run_count[r] == 0) continue;
                rt.begin[rt.n] = run_begin[r];
                rt.count[rt.n] = run_count[r];
                rt.first_block[rt.n + 1] = rt.first_block[rt.n] + (run_count[r] + kChunk - 1) / kChunk;
                if (++rt.n == kMaxParts) flush();
            }
            flush();
        }
    }
    const int rc_launch = rc::check_launch();
    if (rc_launch != RC_OK) return rc_launch;
    if (mean && !(flags & RC_VOXEL_NO_NORMALIZE) && nvox > 0 && F > 0)
        return rc_voxel_normalize(static_cast<float*>(grid), counts, 0, nvox, F, device, stream);
    return RC_OK;
}

}  // extern "C"
