// Point-cloud voxelisation for sm_100a: sort-free binning (pass 1) and mean normalisation
// (pass 2).
//
// Pass 1.  A warp takes 128 consecutive points.  Their packed xyz (1536 contiguous bytes)
// is fetched with three fully coalesced 16-byte loads per lane, parked in the warp's slice
// of shared memory and read back as point (i*32 + lane), i = 0..3 — a stride of three
// words, which is bank-conflict free — so that every later access of the warp (feature
// rows, atomics) is issued for 32 consecutive points.  The voxel id follows the
// reference's arithmetic exactly, in IEEE fp32:
//   v = floor((p - grid_min) / voxel_size) per axis, dropped unless 0 <= v < g on every axis,
//   id = vz*gx*gy + vy*gx + vx
//   (robocache/csrc/cuda/voxelize_kernel.cu:43-61, robocache/validation/cpu_reference.hpp:151-174)
// Scatter: count -> one reduction (no return value) per point or per group of equal ids in
// the warp; occupancy -> a plain store of 1 (every writer stores the same value, no atomic
// needed); mean -> one 16-byte vector reduction per 4 feature channels plus the count.
//
// Pass 2 reads the count plane four voxels per thread and scales the feature sums of
// occupied voxels by 1.0f / count (robocache/csrc/cuda/voxelize_kernel.cu:145-163).
#include "voxel_common.cuh"

#include <atomic>
#include <mutex>

namespace {

using namespace rc::vox;

// Zero-fill for small grids (latency regime): lets the scatter kernel that follows be scheduled
// right away, so that its point loads and voxel-id arithmetic overlap this fill.
__global__ void __launch_bounds__(kThreads) voxel_zero_kernel(unsigned char* __restrict__ p, long long bytes,
                                                              const int* __restrict__ gate = nullptr, int gate_want = 0) {
    grid_dependency_release();
    if (gate != nullptr && *gate != gate_want) return;
    const long long n16 = bytes >> 4;
    uint4* p16 = reinterpret_cast<uint4*>(p);
    const long long stride = static_cast<long long>(gridDim.x) * kThreads;
    for (long long i = blockIdx.x * static_cast<long long>(kThreads) + threadIdx.x; i < n16; i += stride)
        p16[i] = make_uint4(0u, 0u, 0u, 0u);
    if (blockIdx.x == 0)
        for (long long i = (n16 << 4) + threadIdx.x; i < bytes; i += kThreads) p[i] = 0;
}

// Scatter of one point tile.  `id_lo/id_hi` restrict the pass to a slab of voxel ids (a
// contiguous range of the grid in memory); points outside the slab are skipped in this pass.
template <int MODE, bool AGG>
__global__ void __launch_bounds__(kThreads)
voxel_bin_kernel(const float* __restrict__ pts, const float* __restrict__ feats, void* __restrict__ grid_v,
                 int* __restrict__ counts, long long N, int F, VoxelGeom g, bool pts_aligned,
                 long long id_lo, long long id_hi, const int* __restrict__ gate, int gate_want) {
    __shared__ __align__(16) float s_xyz[kThreads / 32][kPointsPerWarp * 3];
    if (gate != nullptr && *gate != gate_want) return;  // this variant was not chosen by the order probe
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const long long ntiles = (N + kPointsPerWarp - 1) / kPointsPerWarp;
    const long long warps_total = static_cast<long long>(gridDim.x) * (kThreads / 32);
    const bool whole_grid = (id_lo <= 0) && (id_hi >= static_cast<long long>(g.gx) * g.gy * g.gz);

    const long long tile0 = static_cast<long long>(blockIdx.x) * (kThreads / 32) + warp;
    float4 ahead[3];  // coordinates of the next fast tile, requested one iteration early
    if (pts_aligned && tile0 < ntiles && (tile0 + 1) * kPointsPerWarp <= N) tile_issue(pts, tile0 * kPointsPerWarp, lane, ahead);
    for (long long tile = tile0; tile < ntiles; tile += warps_total) {
        const long long base = tile * kPointsPerWarp;
        const bool full = base + kPointsPerWarp <= N;

        // mean mode, four channels, single pass: the feature rows are requested together with
        // the coordinates so that every load of the tile is in flight at once
        float4 fv[kPointsPerLane];
        const bool eager = (MODE == kMean) && (F == 4) && full && whole_grid;
        if (eager) {
#pragma unroll
            for (int i = 0; i < kPointsPerLane; ++i)
                fv[i] = __ldcs(reinterpret_cast<const float4*>(feats) + base + i * 32 + lane);
        }

        float x[kPointsPerLane], y[kPointsPerLane], z[kPointsPerLane];
        if (pts_aligned && full) {
            float4 cur[3] = {ahead[0], ahead[1], ahead[2]};
            const long long next = tile + warps_total;
            if (next < ntiles && (next + 1) * kPointsPerWarp <= N) tile_issue(pts, next * kPointsPerWarp, lane, ahead);
            tile_unpack(cur, s_xyz[warp], lane, x, y, z);
        } else {
            tile_load_slow(pts, base, N, lane, x, y, z);
        }

        long long id[kPointsPerLane];
#pragma unroll
        for (int i = 0; i < kPointsPerLane; ++i) {
            id[i] = voxel_id(x[i], y[i], z[i], g);
            if (!whole_grid && (id[i] < id_lo || id[i] >= id_hi)) id[i] = -1;
        }

        grid_dependency_wait();  // the grid may still be being cleared by the preceding launch

        if (MODE == kOccupancy) {
            int* grid = static_cast<int*>(grid_v);
#pragma unroll
            for (int i = 0; i < kPointsPerLane; ++i)
                if (id[i] >= 0) grid[id[i]] = 1;
        } else if (MODE == kOccupancyU8) {
            unsigned char* grid = static_cast<unsigned char*>(grid_v);
#pragma unroll
            for (int i = 0; i < kPointsPerLane; ++i)
                if (id[i] >= 0) grid[id[i]] = 1;
        } else if (MODE == kCount) {
            int* grid = static_cast<int*>(grid_v);
#pragma unroll
            for (int i = 0; i < kPointsPerLane; ++i) {
                if (AGG) {
                    // lanes holding the same voxel elect their lowest lane to add the group size
                    const unsigned int peers = __match_any_sync(0xffffffffu, id[i]);
                    if (id[i] >= 0 && lane == (__ffs(peers) - 1)) atomicAdd(grid + id[i], __popc(peers));
                } else {
                    if (id[i] >= 0) atomicAdd(grid + id[i], 1);
                }
            }
        } else if (MODE == kMean) {
            float* grid = static_cast<float*>(grid_v);
#pragma unroll
            for (int i = 0; i < kPointsPerLane; ++i) {
                const long long pi = base + i * 32 + lane;
                if (id[i] < 0) continue;
                const float* f = feats + pi * F;
                float* o = grid + id[i] * F;
                if (eager) {
                    red_add_v4(o, fv[i]);
                } else if ((F & 3) == 0) {
                    for (int c = 0; c < F; c += 4) red_add_v4(o + c, __ldcs(reinterpret_cast<const float4*>(f + c)));
                } else if ((F & 1) == 0) {
                    for (int c = 0; c < F; c += 2) red_add_v2(o + c, __ldcs(reinterpret_cast<const float2*>(f + c)));
                } else {
                    for (int c = 0; c < F; ++c) atomicAdd(o + c, __ldg(f + c));
                }
                atomicAdd(counts + id[i], 1);
            }
        } else {  // kMax: running maximum kept as an ordered integer, decoded by the fix-up pass
            int* grid = static_cast<int*>(grid_v);
#pragma unroll
            for (int i = 0; i < kPointsPerLane; ++i) {
                const long long pi = base + i * 32 + lane;
                if (id[i] < 0) continue;
                for (int c = 0; c < F; ++c) atomicMax(grid + id[i] * F + c, float_ordered(__ldg(feats + pi * F + c)));
            }
        }
    }
}

// ---------------------------------------------------------------- two-phase scatter for large sparse grids
//
// When the accumulators of a grid do not fit in L2, an atomic that misses waits for a DRAM
// sector, and the scatter runs at a fraction of the rate it reaches on an L2-resident grid.
// Phase 1 writes the voxel id of every point once (4 bytes per point, -1 for dropped points).
// Phase 2 runs P passes over those ids; pass p scatters only the points whose id falls into the
// p-th contiguous slab of the grid, so the sectors it touches stay resident.  Re-reading ids costs
// 4 bytes per point and pass instead of the 12-byte coordinates.

__global__ void __launch_bounds__(kThreads)
voxel_ids_kernel(const float* __restrict__ pts, long long N, VoxelGeom g, bool pts_aligned, int* __restrict__ ids,
                 const int* __restrict__ gate, int gate_want) {
    __shared__ __align__(16) float s_xyz[kThreads / 32][kPointsPerWarp * 3];
    if (gate != nullptr && *gate != gate_want) return;
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const long long ntiles = (N + kPointsPerWarp - 1) / kPointsPerWarp;
    const long long warps_total = static_cast<long long>(gridDim.x) * (kThreads / 32);
    const long long tile0 = static_cast<long long>(blockIdx.x) * (kThreads / 32) + warp;
    float4 ahead[3];
    if (pts_aligned && tile0 < ntiles && (tile0 + 1) * kPointsPerWarp <= N) tile_issue(pts, tile0 * kPointsPerWarp, lane, ahead);
    for (long long tile = tile0; tile < ntiles; tile += warps_total) {
        const long long base = tile * kPointsPerWarp;
        float x[kPointsPerLane], y[kPointsPerLane], z[kPointsPerLane];
        if (pts_aligned && base + kPointsPerWarp <= N) {
            float4 cur[3] = {ahead[0], ahead[1], ahead[2]};
            const long long next = tile + warps_total;
            if (next < ntiles && (next + 1) * kPointsPerWarp <= N) tile_issue(pts, next * kPointsPerWarp, lane, ahead);
            tile_unpack(cur, s_xyz[warp], lane, x, y, z);
        } else {
            tile_load_slow(pts, base, N, lane, x, y, z);
        }
#pragma unroll
        for (int i = 0; i < kPointsPerLane; ++i) {
            const long long pi = base + i * 32 + lane;
            if (pi < N) __stcs(ids + pi, static_cast<int>(voxel_id(x[i], y[i], z[i], g)));
        }
    }
}

// Order probe.  Whether slab passes pay off depends on the order of the points: a spatially coherent
// stream (a scan, cluster after cluster) keeps its accumulators in L2 by itself and is fastest in one
// pass, an iid stream is not.  One CTA looks at kProbeTiles tiles spread over the cloud and counts how
// often two consecutive points fall into the same 1/64 slab of the grid; *flag = 1 (coherent) if at
// least 15 % do.  The kernels of both strategies are launched behind it and the ones that were not
// chosen return at once, so the decision never leaves the device.
constexpr int kProbeTiles = 64;
__global__ void __launch_bounds__(1024)
voxel_order_probe_kernel(const float* __restrict__ pts, long long N, VoxelGeom g, long long V, int* __restrict__ flag) {
    __shared__ int s_same, s_pairs;
    if (threadIdx.x == 0) { s_same = 0; s_pairs = 0; }
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const long long ntiles = N / kPointsPerWarp;  // full tiles only
    const long long step = ntiles > kProbeTiles ? ntiles / kProbeTiles : 1;
    int same = 0, pairs = 0;
    for (long long t = warp; t < kProbeTiles && t * step < ntiles; t += 32) {
        const long long base = t * step * kPointsPerWarp;
        float x[kPointsPerLane], y[kPointsPerLane], z[kPointsPerLane];
        tile_load_slow(pts, base, N, lane, x, y, z);
#pragma unroll
        for (int i = 0; i < kPointsPerLane; ++i) {
            const long long id = voxel_id(x[i], y[i], z[i], g);
            const int slab = (id < 0) ? -1 : static_cast<int>(id * 64 / V);
            const int next = __shfl_down_sync(0xffffffffu, slab, 1);
            const bool ok = lane < 31 && slab >= 0 && next >= 0;
            pairs += __popc(__ballot_sync(0xffffffffu, ok));
            same += __popc(__ballot_sync(0xffffffffu, ok && slab == next));
        }
    }
    if (lane == 0) { atomicAdd(&s_same, same); atomicAdd(&s_pairs, pairs); }
    __syncthreads();
    if (threadIdx.x == 0) *flag = (s_pairs > 0 && 100ll * s_same >= 15ll * s_pairs) ? 1 : 0;
}


// ids is 16-byte aligned.  Per step a warp reads 256 consecutive ids (two 16-byte loads per lane),
// compacts the points of the current slab into its shared-memory queue with ballots, and then
// scatters the queue with all lanes busy: a pass costs one cheap scan of the ids plus only its own
// share of the feature gathers and atomics.
template <int MODE>
__global__ void __launch_bounds__(kThreads)
voxel_scatter_ids_kernel(const int* __restrict__ ids, const float* __restrict__ feats, void* __restrict__ grid_v,
                         int* __restrict__ counts, long long N, int F, int id_lo, int id_hi,
                         const int* __restrict__ gate, int gate_want) {
    __shared__ int s_id[kThreads / 32][256];
    if (gate != nullptr && *gate != gate_want) return;
    __shared__ int s_pt[kThreads / 32][256];   // point index relative to the warp's step base
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const unsigned int lt_mask = (1u << lane) - 1u;
    const long long steps = (N + 255) >> 8;
    const long long warps_total = static_cast<long long>(gridDim.x) * (kThreads / 32);
    const unsigned int span = static_cast<unsigned int>(id_hi - id_lo);
    int* qid = s_id[warp];
    int* qpt = s_pt[warp];
    for (long long step = static_cast<long long>(blockIdx.x) * (kThreads / 32) + warp; step < steps; step += warps_total) {
        const long long base = step << 8;
        int v[8];
        if (base + 256 <= N) {
            const int4 a = __ldcs(reinterpret_cast<const int4*>(ids + base) + lane);
            const int4 b = __ldcs(reinterpret_cast<const int4*>(ids + base) + 32 + lane);
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        } else {
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const long long pi = base + (k >> 2) * 128 + lane * 4 + (k & 3);
                v[k] = (pi < N) ? ids[pi] : -1;
            }
        }
        int n = 0;
#pragma unroll
        for (int k = 0; k < 8; ++k) {  // one unsigned compare covers id >= lo, id < hi and id == -1
            const bool in = static_cast<unsigned int>(v[k] - id_lo) < span;
            const unsigned int m = __ballot_sync(0xffffffffu, in);
            if (in) {
                const int slot = n + __popc(m & lt_mask);
                qid[slot] = v[k];
                qpt[slot] = (k >> 2) * 128 + lane * 4 + (k & 3);
            }
            n += __popc(m);
        }
        __syncwarp();
        for (int j = lane; j < n; j += 32) scatter_one<MODE>(qid[j], base + qpt[j], feats, grid_v, counts, F);
        __syncwarp();
    }
}

// mean pass 2, wide form: counts + v0 is 16-byte aligned and (v1 - v0) % 4 == 0.  Per step a warp reads
// 256 consecutive counters (two 16-byte loads per lane), queues the occupied voxels among them in
// shared memory with ballots, and rescales the queued voxels with all lanes busy and independent
// loads in flight; empty regions of a sparse grid cost one streaming read of the counter plane.
template <bool VEC4>
__global__ void __launch_bounds__(kThreads)
voxel_normalize_wide_kernel(float* __restrict__ grid, const int* __restrict__ counts, long long v0, long long v1, int F,
                            const int* __restrict__ gate, int gate_want) {
    __shared__ int s_vox[kThreads / 32][256];
    __shared__ int s_cnt[kThreads / 32][256];
    if (gate != nullptr && *gate != gate_want) return;
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const unsigned int lt_mask = (1u << lane) - 1u;
    const long long nvox = v1 - v0;
    const long long steps = (nvox + 255) >> 8;
    const long long warps_total = static_cast<long long>(gridDim.x) * (kThreads / 32);
    int* qv = s_vox[warp];
    int* qc = s_cnt[warp];
    for (long long step = static_cast<long long>(blockIdx.x) * (kThreads / 32) + warp; step < steps; step += warps_total) {
        const long long base = v0 + (step << 8);
        const long long left = v1 - base;  // > 0, multiple of 4
        int c[8];
        const int4 z = make_int4(0, 0, 0, 0);
        const int4 a = (lane * 4 < left) ? __ldcs(reinterpret_cast<const int4*>(counts + base) + lane) : z;
        const int4 b = (128 + lane * 4 < left) ? __ldcs(reinterpret_cast<const int4*>(counts + base) + 32 + lane) : z;
        c[0] = a.x; c[1] = a.y; c[2] = a.z; c[3] = a.w; c[4] = b.x; c[5] = b.y; c[6] = b.z; c[7] = b.w;
        int n = 0;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const bool occ = c[k] > 0;  // empty voxels stay exactly 0
            const unsigned int m = __ballot_sync(0xffffffffu, occ);
            if (occ) {
                const int slot = n + __popc(m & lt_mask);
                qv[slot] = (k >> 2) * 128 + lane * 4 + (k & 3);
                qc[slot] = c[k];
            }
            n += __popc(m);
        }
        __syncwarp();
#pragma unroll 2
        for (int j = lane; j < n; j += 32) {
            const float inv = __fdiv_rn(1.0f, static_cast<float>(qc[j]));
            float* o = grid + (base + qv[j]) * F;
            if (VEC4) {
                for (int f = 0; f < F; f += 4) {
                    float4 sgl = *reinterpret_cast<float4*>(o + f);
                    sgl.x = __fmul_rn(sgl.x, inv); sgl.y = __fmul_rn(sgl.y, inv);
                    sgl.z = __fmul_rn(sgl.z, inv); sgl.w = __fmul_rn(sgl.w, inv);
                    *reinterpret_cast<float4*>(o + f) = sgl;
                }
            } else {
                for (int f = 0; f < F; ++f) o[f] = __fmul_rn(o[f], inv);
            }
        }
        __syncwarp();
    }
}

// mean pass 2 for four channels, streaming form: counts + v0 and grid are 16-byte aligned, (v1 - v0) % 4 == 0.  A warp
// reads 512 consecutive counters per step (four 16-byte loads per lane, all in flight together) and rescales the
// occupied voxels among its own sixteen; on a sparse grid almost all of the work is the counter stream.
__global__ void __launch_bounds__(kThreads)
voxel_normalize_stream_kernel(float4* __restrict__ grid4, const int* __restrict__ counts, long long v0, long long v1,
                              const int* __restrict__ gate, int gate_want) {
    if (gate != nullptr && *gate != gate_want) return;
    const int lane = threadIdx.x & 31;
    const long long warps_total = static_cast<long long>(gridDim.x) * (kThreads / 32);
    const long long steps = (v1 - v0 + 511) >> 9;
    for (long long step = static_cast<long long>(blockIdx.x) * (kThreads / 32) + (threadIdx.x >> 5); step < steps; step += warps_total) {
        const long long base = v0 + (step << 9) + lane * 4;
        int4 c[4];
#pragma unroll
        for (int k = 0; k < 4; ++k)
            c[k] = (base + k * 128 < v1) ? __ldcs(reinterpret_cast<const int4*>(counts + base + k * 128)) : make_int4(0, 0, 0, 0);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int cc[4] = {c[k].x, c[k].y, c[k].z, c[k].w};
            if ((cc[0] | cc[1] | cc[2] | cc[3]) == 0) continue;     // counters are never negative
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (cc[j] > 0) {                                    // empty voxels stay exactly 0
                    const float inv = __fdiv_rn(1.0f, static_cast<float>(cc[j]));
                    float4* o = grid4 + base + k * 128 + j;
                    float4 x = *o;
                    x.x = __fmul_rn(x.x, inv); x.y = __fmul_rn(x.y, inv);
                    x.z = __fmul_rn(x.z, inv); x.w = __fmul_rn(x.w, inv);
                    *o = x;
                }
            }
        }
    }
}

// mean pass 2, one voxel per thread: ragged ends of a range and unaligned buffers
__global__ void __launch_bounds__(kThreads)
voxel_normalize_scalar_kernel(float* __restrict__ grid, const int* __restrict__ counts, long long v0, long long v1, int F,
                              const int* __restrict__ gate, int gate_want) {
    if (gate != nullptr && *gate != gate_want) return;
    const long long v = v0 + blockIdx.x * static_cast<long long>(kThreads) + threadIdx.x;
    if (v >= v1) return;
    const int c = counts[v];
    if (c <= 0) return;
    const float inv = __fdiv_rn(1.0f, static_cast<float>(c));
    for (int f = 0; f < F; ++f) grid[v * F + f] = __fmul_rn(grid[v * F + f], inv);
}

// max mode set-up and fix-up: the grid holds ordered integers while points are binned
constexpr int kMaxEmpty = static_cast<int>(0x80000000u);
__global__ void __launch_bounds__(kThreads) voxel_max_fill_kernel(int* __restrict__ grid, long long n) {
    for (long long i = blockIdx.x * static_cast<long long>(kThreads) + threadIdx.x; i < n;
         i += static_cast<long long>(gridDim.x) * kThreads)
        grid[i] = kMaxEmpty;
}
__global__ void __launch_bounds__(kThreads) voxel_max_decode_kernel(int* __restrict__ grid, long long n) {
    for (long long i = blockIdx.x * static_cast<long long>(kThreads) + threadIdx.x; i < n;
         i += static_cast<long long>(gridDim.x) * kThreads) {
        const int o = grid[i];
        grid[i] = (o == kMaxEmpty) ? 0 : ((o >= 0) ? o : (o ^ 0x7fffffff));  // empty voxel -> 0.0f
    }
}

template <int MODE, bool AGG>
void launch_bin_one(bool overlap_prev, unsigned int blocks, cudaStream_t st, const float* pts, const float* feats,
                    void* grid, int* counts, long long N, int F, const VoxelGeom& g, bool aligned, long long id_lo,
                    long long id_hi, const int* gate, int gate_want) {
    if (overlap_prev) {
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(blocks);
        cfg.blockDim = dim3(kThreads);
        cfg.dynamicSmemBytes = 0;
        cfg.stream = st;
        cudaLaunchAttribute attr{};
        attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr.val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        if (cudaLaunchKernelEx(&cfg, voxel_bin_kernel<MODE, AGG>, pts, feats, grid, counts, N, F, g, aligned, id_lo,
                               id_hi, gate, gate_want) == cudaSuccess)
            return;
        cudaGetLastError();  // attribute refused: fall through to an ordinary launch
    }
    voxel_bin_kernel<MODE, AGG><<<blocks, kThreads, 0, st>>>(pts, feats, grid, counts, N, F, g, aligned, id_lo, id_hi,
                                                             gate, gate_want);
}

template <int MODE>
void launch_bin(bool agg, bool overlap_prev, unsigned int blocks, cudaStream_t st, const float* pts, const float* feats,
                void* grid, int* counts, long long N, int F, const VoxelGeom& g, bool aligned, long long id_lo,
                long long id_hi, const int* gate = nullptr, int gate_want = 0) {
    if (agg) launch_bin_one<MODE, true>(overlap_prev, blocks, st, pts, feats, grid, counts, N, F, g, aligned, id_lo, id_hi, gate, gate_want);
    else     launch_bin_one<MODE, false>(overlap_prev, blocks, st, pts, feats, grid, counts, N, F, g, aligned, id_lo, id_hi, gate, gate_want);
}

// ---------------------------------------------------------------- allocation-free mean mode
//
// Count plane for rc_voxelize_mean_static.  It lives in the library image: every GPU that
// loads the library holds these 8 MiB until the process exits, and every call on a device
// shares them.
constexpr long long kStaticMaxVoxels = RC_STATIC_MAX_VOXELS;
static __device__ __align__(256) int g_static_counts[kStaticMaxVoxels];

// Device address of g_static_counts on `device`, which must be current.  In host code the
// array's name is only a handle for the runtime, never an address a kernel may use, so the
// address is asked for once per device and remembered.
int static_counts_address(int device, int** out) {
    static std::mutex mu;
    static int* known[64] = {};
    if (device < 0 || device >= 64) return RC_ERR_BAD_DEVICE;
    std::lock_guard<std::mutex> lock(mu);
    if (known[device] == nullptr) {
        void* p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_static_counts);
        if (e != cudaSuccess) return rc::cuda_fail(e);
        known[device] = static_cast<int*>(p);
    }
    *out = known[device];
    return RC_OK;
}

// slabs of the run path: RC_OPT_VOXEL_PASSES when set, else the default
int mean_runs_parts() {
    const int forced = rc::g_voxel_passes.load(std::memory_order_relaxed);
    if (forced > 1) return forced < kMeanRunsMaxParts ? forced : kMeanRunsMaxParts;
    return kMeanRunsParts;
}

// Pass 2 over voxels [voxel_begin, voxel_end) on the current device; with a gate the kernels return at once
// unless *gate == gate_want.
int normalize_range(float* grid, const int* counts, long long voxel_begin, long long voxel_end, int F, int device,
                    cudaStream_t st, const int* gate, int gate_want) {
    // [voxel_begin, head) and [body_end, voxel_end) go voxel by voxel; the body, whose count
    // pointer is 16-byte aligned and whose length is a multiple of four, goes four per thread
    long long head = voxel_begin;
    while (head < voxel_end && !rc::aligned_to(counts + head, 16)) ++head;
    const long long body_end = head + ((voxel_end - head) & ~3ll);
    auto scalar = [&](long long a, long long b) {
        if (b > a) {
            const long long blocks = (b - a + kThreads - 1) / kThreads;
            voxel_normalize_scalar_kernel<<<static_cast<unsigned int>(blocks), kThreads, 0, st>>>(grid, counts, a, b, F, gate, gate_want);
        }
    };
    if ((voxel_end - voxel_begin + kThreads - 1) / kThreads >= (1ll << 31)) return RC_ERR_TOO_LARGE;
    scalar(voxel_begin, head);
    if (body_end > head) {
        long long blocks = (((body_end - head) + 255) / 256 + kThreads / 32 - 1) / (kThreads / 32);
        const long long cap = 16ll * rc::sm_count(device);
        if (blocks > cap) blocks = cap;
        const unsigned int nb = static_cast<unsigned int>(blocks);
        if (F == 4 && rc::aligned_to(grid, 16)) {
            long long sb = (((body_end - head) + 511) / 512 + kThreads / 32 - 1) / (kThreads / 32);
            if (sb > cap) sb = cap;
            voxel_normalize_stream_kernel<<<static_cast<unsigned int>(sb), kThreads, 0, st>>>(reinterpret_cast<float4*>(grid), counts, head,
                                                                                            body_end, gate, gate_want);
        } else if ((F & 3) == 0 && rc::aligned_to(grid, 16))
            voxel_normalize_wide_kernel<true><<<nb, kThreads, 0, st>>>(grid, counts, head, body_end, F, gate, gate_want);
        else
            voxel_normalize_wide_kernel<false><<<nb, kThreads, 0, st>>>(grid, counts, head, body_end, F, gate, gate_want);
    }
    scalar(body_end, voxel_end);
    return rc::check_launch();
}

}  // namespace

extern "C" {

int rc_voxel_normalize(float* grid, const int32_t* counts, int64_t voxel_begin, int64_t voxel_end,
                       int32_t F, int device, void* stream) {
    if (voxel_begin < 0 || voxel_end < voxel_begin || F < 0) return RC_ERR_BAD_SHAPE;
    if (voxel_end == voxel_begin || F == 0) return RC_OK;
    if (grid == nullptr || counts == nullptr) return RC_ERR_NULL_POINTER;
    if (!rc::aligned_to(grid, 4) || !rc::aligned_to(counts, 4)) return RC_ERR_BAD_ALIGNMENT;
    rc::DeviceScope scope(device);
    if (scope.status() != RC_OK) return scope.status();
    return normalize_range(grid, counts, voxel_begin, voxel_end, F, device, static_cast<cudaStream_t>(stream), nullptr, 0);
}

int rc_voxelize(const float* points, const float* features, void* grid, int32_t* counts, int64_t N,
                int32_t F, const float grid_min_host[3], float voxel_size,
                const int32_t grid_size_host[3], int mode, uint32_t flags, int device, void* stream) {
    return rc_voxelize_ex(points, features, grid, counts, N, F, grid_min_host, voxel_size, grid_size_host, mode, flags,
                          nullptr, 0, device, stream);
}

uint64_t rc_voxelize_scratch_bytes(int64_t N, int32_t F, const int32_t grid_size_host[3], int mode) {
    if (grid_size_host == nullptr || N <= 0) return 0;
    if (mode != RC_VOXEL_MEAN && mode != RC_VOXEL_COUNT) return 0;
    const double cells = static_cast<double>(grid_size_host[0]) * grid_size_host[1] * grid_size_host[2];
    if (cells <= 0 || cells >= 2147483648.0) return 0;
    const double acc_bytes = cells * 4.0 * (mode == RC_VOXEL_MEAN ? (1 + (F > 0 ? F : 0)) : 1);
    const bool forced = rc::g_voxel_passes.load(std::memory_order_relaxed) > 1;
    if (acc_bytes <= static_cast<double>(kResidentBytes) && !forced) return 0;  // L2-resident accumulators: one pass
    if (mode == RC_VOXEL_COUNT) return (N >= kProbeMinPoints) ? 16 : 0;     // the order probe's flag
    if (F == 4 && cells < 2147483648.0 && N <= (1ll << 31) - 4096)           // slab-ordered runs + flag
        return mean_runs_scratch_bytes(N, static_cast<long long>(cells), mean_runs_parts()) + 256u;
    return ((static_cast<uint64_t>(N) * 4u + 15u) & ~static_cast<uint64_t>(15)) + 16u;  // ids + flag
}

int rc_voxelize_ex(const float* points, const float* features, void* grid, int32_t* counts, int64_t N,
                   int32_t F, const float grid_min_host[3], float voxel_size,
                   const int32_t grid_size_host[3], int mode, uint32_t flags, void* scratch, uint64_t scratch_bytes,
                   int device, void* stream) {
    if (mode < RC_VOXEL_COUNT || mode > RC_VOXEL_OCCUPANCY_U8) return RC_ERR_BAD_MODE;
    if (grid_min_host == nullptr || grid_size_host == nullptr || grid == nullptr) return RC_ERR_NULL_POINTER;
    if (N < 0 || F < 0) return RC_ERR_BAD_SHAPE;
    if (!(voxel_size > 0.0f) || !(voxel_size <= 3.0e38f)) return RC_ERR_BAD_VALUE;
    const bool feat_mode = (mode == RC_VOXEL_MEAN || mode == RC_VOXEL_MAX);
    VoxelGeom g;
    g.minx = grid_min_host[0]; g.miny = grid_min_host[1]; g.minz = grid_min_host[2];
    g.vs = voxel_size;
    g.gx = grid_size_host[0]; g.gy = grid_size_host[1]; g.gz = grid_size_host[2];
    if (g.gx < 0 || g.gy < 0 || g.gz < 0) return RC_ERR_BAD_SHAPE;
    if (g.gx >= (1 << 24) || g.gy >= (1 << 24) || g.gz >= (1 << 24)) return RC_ERR_TOO_LARGE;
    g.fgx = static_cast<float>(g.gx); g.fgy = static_cast<float>(g.gy); g.fgz = static_cast<float>(g.gz);
    g.inv_vs = host_reciprocal(voxel_size);
    const long long V = static_cast<long long>(g.gx) * g.gy * g.gz;  // < 2^72 impossible: each < 2^24 -> check below
    if (static_cast<double>(g.gx) * g.gy * g.gz * (feat_mode ? (F > 0 ? F : 1) : 1) >= 1099511627776.0)
        return RC_ERR_TOO_LARGE;
    if (feat_mode && N > 0 && F > 0 && features == nullptr) return RC_ERR_BAD_MODE;
    if (mode == RC_VOXEL_MEAN && counts == nullptr) return RC_ERR_NULL_POINTER;
    if (N > 0 && points == nullptr) return RC_ERR_NULL_POINTER;
    if (!rc::aligned_to(points, 4) || !rc::aligned_to(features, 4) || !rc::aligned_to(counts, 4))
        return RC_ERR_BAD_ALIGNMENT;
    if (mode != RC_VOXEL_OCCUPANCY_U8 && !rc::aligned_to(grid, 4)) return RC_ERR_BAD_ALIGNMENT;

    rc::DeviceScope scope(device);
    if (scope.status() != RC_OK) return scope.status();
    cudaStream_t st = static_cast<cudaStream_t>(stream);

    const long long cells = feat_mode ? V * F : V;
    const size_t cell_bytes = (mode == RC_VOXEL_OCCUPANCY_U8) ? 1 : 4;
    const long long fill_blocks_ll = (cells + kThreads - 1) / kThreads;
    const unsigned int fill_blocks =
        static_cast<unsigned int>(fill_blocks_ll < 64ll * rc::sm_count(device) ? (fill_blocks_ll > 0 ? fill_blocks_ll : 1)
                                                                           : 64ll * rc::sm_count(device));
    // Mean mode, four channels, accumulators beyond L2, enough scratch: slab-ordered runs (voxel_runs.cu) between
    // one clear and one normalise pass.  With points in coherent order (decided on the device by the order probe)
    // one plain pass is faster; its kernel is enqueued too and the strategy not chosen returns at once.
    {
        const int forced = rc::g_voxel_passes.load(std::memory_order_relaxed);
        const double acc_bytes = static_cast<double>(V) * 4.0 * (1 + F);
        const int parts = mean_runs_parts();
        const uint64_t need = (mode == RC_VOXEL_MEAN && F == 4 && V > 0 && V < (1ll << 31) && N > 0 && N <= (1ll << 31) - 4096)
                                  ? mean_runs_scratch_bytes(N, V, parts) + 256u : 0;
        if (need > 0 && (forced > 1 || (forced == 0 && acc_bytes > static_cast<double>(kResidentBytes))) &&
            scratch != nullptr && rc::aligned_to(scratch, 256) && scratch_bytes >= need && rc::aligned_to(features, 16) &&
            rc::aligned_to(grid, 16) && features != nullptr) {
            if (flags & RC_VOXEL_ZERO_INIT) {
                RC_CUDA_TRY(cudaMemsetAsync(grid, 0, static_cast<size_t>(V) * 16, st));
                RC_CUDA_TRY(cudaMemsetAsync(counts, 0, static_cast<size_t>(V) * 4, st));
            }
            int* flag = nullptr;
            if (forced == 0 && N >= kProbeMinPoints) {
                flag = reinterpret_cast<int*>(static_cast<unsigned char*>(scratch) + need - 256u);
                voxel_order_probe_kernel<<<1, 1024, 0, st>>>(points, N, g, V, flag);
                const long long cap = 16ll * rc::sm_count(device);
                long long blocks = (N + kPointsPerBlock - 1) / kPointsPerBlock;
                if (blocks > cap) blocks = cap;
                launch_bin<kMean>(false, false, static_cast<unsigned int>(blocks), st, points, features, grid, counts, N, F, g,
                                  rc::aligned_to(points, 16), 0, V, flag, 1);
            }
            const int rc_runs = mean_runs_launch(points, features, static_cast<float*>(grid), counts, N, g, V, parts, scratch,
                                                 flag, 0, device, st);
            if (rc_runs != RC_OK) return rc_runs;
            if (!(flags & RC_VOXEL_NO_NORMALIZE))
                return normalize_range(static_cast<float*>(grid), counts, 0, V, F, device, st, nullptr, 0);
            return RC_OK;
        }
    }
    bool overlap_fill = false;
    if (mode == RC_VOXEL_MAX) {
        // max mode always starts from "empty": the caller's buffer content is never an operand
        if (cells > 0) voxel_max_fill_kernel<<<fill_blocks, kThreads, 0, st>>>(static_cast<int*>(grid), cells);
    } else if ((flags & RC_VOXEL_ZERO_INIT) && !feat_mode && cells > 0 &&
               static_cast<size_t>(cells) * cell_bytes <= kSmallGridBytes && rc::aligned_to(grid, 16)) {
        // small grid: own fill kernel, and the scatter below is allowed to start before it has finished
        const long long fb = (static_cast<long long>(cells) * cell_bytes / 16 + kThreads - 1) / kThreads;
        const long long fcap = 8ll * rc::sm_count(device);
        voxel_zero_kernel<<<static_cast<unsigned int>(fb < 1 ? 1 : (fb > fcap ? fcap : fb)), kThreads, 0, st>>>(
            static_cast<unsigned char*>(grid), static_cast<long long>(cells) * cell_bytes);
        overlap_fill = true;
    } else if (flags & RC_VOXEL_ZERO_INIT) {
        if (cells > 0) RC_CUDA_TRY(cudaMemsetAsync(grid, 0, static_cast<size_t>(cells) * cell_bytes, st));
        if (mode == RC_VOXEL_MEAN && V > 0) RC_CUDA_TRY(cudaMemsetAsync(counts, 0, static_cast<size_t>(V) * 4, st));
    }

    if (N > 0 && V > 0 && !(feat_mode && F == 0)) {
        long long blocks = (N + kPointsPerBlock - 1) / kPointsPerBlock;
        const long long cap = 16ll * rc::sm_count(device);  // two waves of resident CTAs; warps stride over tiles
        if (blocks > cap) blocks = cap;
        const unsigned int nb = static_cast<unsigned int>(blocks);
        const bool aligned = rc::aligned_to(points, 16);
        const bool agg = (flags & RC_VOXEL_WARP_AGGREGATE) != 0;
        // vector feature accesses need the feature rows and grid cells aligned to their width
        if (feat_mode) {
            const bool a16 = rc::aligned_to(features, 16) && rc::aligned_to(grid, 16);
            const bool a8 = rc::aligned_to(features, 8) && rc::aligned_to(grid, 8);
            if ((F & 3) == 0 && !a16) return RC_ERR_BAD_ALIGNMENT;
            if ((F & 3) != 0 && (F & 1) == 0 && !a8) return RC_ERR_BAD_ALIGNMENT;
        }
        // Slab passes (RC_OPT_VOXEL_PASSES, 0 = automatic): each pass scatters only into one contiguous
        // range of voxel ids so that the sectors it touches stay resident in L2.
        const int forced = rc::g_voxel_passes.load(std::memory_order_relaxed);
        const bool scatter_mode = (mode == RC_VOXEL_COUNT || mode == RC_VOXEL_MEAN || mode == RC_VOXEL_MAX);
        const double acc_bytes = static_cast<double>(V) * 4.0 * (mode == RC_VOXEL_MEAN ? (1 + F) : (feat_mode ? F : 1));
        const bool big = acc_bytes > static_cast<double>(kResidentBytes);
        const uint64_t ids_bytes = (static_cast<uint64_t>(N) * 4u + 15u) & ~static_cast<uint64_t>(15);
        const bool ids_room = scratch != nullptr && rc::aligned_to(scratch, 16) && scratch_bytes >= ids_bytes && V < (1ll << 31);
        const bool ids_path = (mode == RC_VOXEL_MEAN) && ids_room && (forced > 1 || (forced == 0 && big));
        // automatic choice on large grids: let the order probe pick between one pass and slab passes
        int* flag = nullptr;
        if (forced == 0 && big && N >= kProbeMinPoints && scratch != nullptr && rc::aligned_to(scratch, 16)) {
            if (mode == RC_VOXEL_MEAN && ids_room && scratch_bytes >= ids_bytes + 16)
                flag = reinterpret_cast<int*>(static_cast<unsigned char*>(scratch) + ids_bytes);
            else if (mode == RC_VOXEL_COUNT && scratch_bytes >= 16)
                flag = static_cast<int*>(scratch);
        }
        if (flag != nullptr) voxel_order_probe_kernel<<<1, 1024, 0, st>>>(points, N, g, V, flag);
        int passes = 1;
        if (scatter_mode) {
            if (forced > 0) passes = forced;
            else if (ids_path) passes = kAutoMeanPasses;
            else if (mode == RC_VOXEL_COUNT && big) passes = 2;
        }
        if (passes > V) passes = static_cast<int>(V);
        const long long slab = (V + passes - 1) / passes;
        if (flag != nullptr) {
            // coherent order (flag 1): one pass over the whole grid
            if (mode == RC_VOXEL_MEAN) launch_bin<kMean>(false, false, nb, st, points, features, grid, counts, N, F, g, aligned, 0, V, flag, 1);
            else launch_bin<kCount>(agg, false, nb, st, points, features, grid, counts, N, F, g, aligned, 0, V, flag, 1);
        }
        if (ids_path) {
            int* ids = static_cast<int*>(scratch);
            voxel_ids_kernel<<<nb, kThreads, 0, st>>>(points, N, g, aligned, ids, flag, 0);
            long long sb = (((N + 255) >> 8) + kThreads / 32 - 1) / (kThreads / 32);
            if (sb > cap) sb = cap;
            if (sb < 1) sb = 1;
            for (int ps = 0; ps < passes; ++ps) {
                const long long lo = ps * slab;
                const long long hi = (lo + slab < V) ? lo + slab : V;
                voxel_scatter_ids_kernel<kMean><<<static_cast<unsigned int>(sb), kThreads, 0, st>>>(
                    ids, features, grid, counts, N, F, static_cast<int>(lo), static_cast<int>(hi), flag, 0);
            }
        } else {
            for (int ps = 0; ps < passes; ++ps) {
                const long long lo = (passes == 1) ? 0 : ps * slab;
                const long long hi = (passes == 1) ? V : ((ps + 1) * slab < V ? (ps + 1) * slab : V);
                switch (mode) {
                    case RC_VOXEL_COUNT: launch_bin<kCount>(agg, overlap_fill && ps == 0, nb, st, points, features, grid, counts, N, F, g, aligned, lo, hi, flag, 0); break;
                    case RC_VOXEL_OCCUPANCY: launch_bin<kOccupancy>(false, overlap_fill && ps == 0, nb, st, points, features, grid, counts, N, F, g, aligned, lo, hi); break;
                    case RC_VOXEL_OCCUPANCY_U8: launch_bin<kOccupancyU8>(false, overlap_fill && ps == 0, nb, st, points, features, grid, counts, N, F, g, aligned, lo, hi); break;
                    case RC_VOXEL_MEAN: launch_bin<kMean>(false, overlap_fill && ps == 0, nb, st, points, features, grid, counts, N, F, g, aligned, lo, hi); break;
                    default: launch_bin<kMax>(false, overlap_fill && ps == 0, nb, st, points, features, grid, counts, N, F, g, aligned, lo, hi); break;
                }
            }
        }
    }
    if (mode == RC_VOXEL_MAX && cells > 0) {
        voxel_max_decode_kernel<<<fill_blocks, kThreads, 0, st>>>(static_cast<int*>(grid), cells);
    }
    int rc_launch = rc::check_launch();
    if (rc_launch != RC_OK) return rc_launch;
    if (mode == RC_VOXEL_MEAN && !(flags & RC_VOXEL_NO_NORMALIZE) && V > 0 && F > 0) {
        return rc_voxel_normalize(static_cast<float*>(grid), counts, 0, V, F, device, stream);
    }
    return RC_OK;
}

int rc_voxel_scatter_ids(const int32_t* ids, const float* features, void* grid, int32_t* counts, int64_t M,
                         int32_t F, int64_t id_begin, int64_t id_end, int mode, uint32_t flags, int device,
                         void* stream) {
    if (mode != RC_VOXEL_COUNT && mode != RC_VOXEL_OCCUPANCY && mode != RC_VOXEL_MEAN) return RC_ERR_BAD_MODE;
    if (M < 0 || F < 0 || id_begin < 0 || id_end < id_begin) return RC_ERR_BAD_SHAPE;
    if (id_end >= (1ll << 31)) return RC_ERR_TOO_LARGE;
    const long long nvox = id_end - id_begin;
    const bool mean = (mode == RC_VOXEL_MEAN);
    if (nvox > 0 && (!mean || F > 0) && grid == nullptr) return RC_ERR_NULL_POINTER;
    if (mean && nvox > 0 && counts == nullptr) return RC_ERR_NULL_POINTER;
    if (M > 0 && ids == nullptr) return RC_ERR_NULL_POINTER;
    if (mean && M > 0 && F > 0 && features == nullptr) return RC_ERR_BAD_MODE;
    if (!rc::aligned_to(ids, 16) || !rc::aligned_to(grid, 4) || !rc::aligned_to(counts, 4) || !rc::aligned_to(features, 4))
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
    if (M > 0 && nvox > 0 && !(mean && F == 0)) {
        // the kernel indexes with the global id: hand it the address voxel 0 would have
        const uintptr_t cell = mean ? static_cast<uintptr_t>(F) * 4u : 4u;
        void* grid0 = reinterpret_cast<void*>(reinterpret_cast<uintptr_t>(grid) - static_cast<uintptr_t>(id_begin) * cell);
        int* counts0 = mean ? reinterpret_cast<int*>(reinterpret_cast<uintptr_t>(counts) - static_cast<uintptr_t>(id_begin) * 4u)
                            : nullptr;
        const int forced = rc::g_voxel_passes.load(std::memory_order_relaxed);
        const double acc_bytes = static_cast<double>(nvox) * 4.0 * (mean ? (1 + F) : 1);
        int passes = 1;
        if (forced > 0) passes = forced;
        else if (mode != RC_VOXEL_OCCUPANCY && acc_bytes > static_cast<double>(kResidentBytes))
            passes = static_cast<int>((acc_bytes + kSlabPassBytes - 1) / kSlabPassBytes);
        if (passes > 64) passes = 64;
        if (passes > nvox) passes = static_cast<int>(nvox);
        const long long span = (nvox + passes - 1) / passes;
        long long sb = (((M + 255) >> 8) + kThreads / 32 - 1) / (kThreads / 32);
        const long long cap = 16ll * rc::sm_count(device);
        if (sb > cap) sb = cap;
        const unsigned int nb = static_cast<unsigned int>(sb < 1 ? 1 : sb);
        for (int ps = 0; ps < passes; ++ps) {
            const int lo = static_cast<int>(id_begin + ps * span);
            const int hi = static_cast<int>((id_begin + (ps + 1) * span < id_end) ? id_begin + (ps + 1) * span : id_end);
            if (mode == RC_VOXEL_MEAN)
                voxel_scatter_ids_kernel<kMean><<<nb, kThreads, 0, st>>>(ids, features, grid0, counts0, M, F, lo, hi, nullptr, 0);
            else if (mode == RC_VOXEL_COUNT)
                voxel_scatter_ids_kernel<kCount><<<nb, kThreads, 0, st>>>(ids, features, grid0, counts0, M, F, lo, hi, nullptr, 0);
            else
                voxel_scatter_ids_kernel<kOccupancy><<<nb, kThreads, 0, st>>>(ids, features, grid0, counts0, M, F, lo, hi, nullptr, 0);
        }
    }
    const int rc_launch = rc::check_launch();
    if (rc_launch != RC_OK) return rc_launch;
    if (mean && !(flags & RC_VOXEL_NO_NORMALIZE) && nvox > 0 && F > 0)
        return rc_voxel_normalize(static_cast<float*>(grid), counts, 0, nvox, F, device, stream);
    return RC_OK;
}

// Mean-mode voxelisation for callers that must not allocate device memory: code running
// inside a framework's memory-pool callback or under a real-time loop's "no driver
// allocation after start-up" rule, or a host that was only handed the input and output
// buffers.  Mean mode needs one int32 counter per voxel next to the output; here that plane
// is the file-scope array above instead of a caller buffer, so nothing is allocated, by this
// function or on its behalf.  The grid and the counters are cleared on `stream` first, then
// the points are binned and the sums normalised exactly as rc_voxelize does.
int rc_voxelize_mean_static(const float* points, const float* features, float* grid, int64_t N, int32_t F,
                            const float grid_min_host[3], float voxel_size, const int32_t grid_size_host[3],
                            int device, void* stream) {
    if (grid_size_host == nullptr) return RC_ERR_NULL_POINTER;
    for (int a = 0; a < 3; ++a)
        if (grid_size_host[a] < 0) return RC_ERR_BAD_SHAPE;
    const double voxels = static_cast<double>(grid_size_host[0]) * grid_size_host[1] * grid_size_host[2];
    if (voxels > static_cast<double>(kStaticMaxVoxels)) return RC_ERR_TOO_LARGE;  // the counter plane is fixed size
    rc::DeviceScope scope(device);
    if (scope.status() != RC_OK) return scope.status();
    int* counts = nullptr;
    const int rc_addr = static_counts_address(device, &counts);
    if (rc_addr != RC_OK) return rc_addr;
    // RC_VOXEL_ZERO_INIT clears the grid and the shared counters, which keep the previous call's values
    return rc_voxelize(points, features, grid, counts, N, F, grid_min_host, voxel_size, grid_size_host,
                       RC_VOXEL_MEAN, RC_VOXEL_ZERO_INIT, device, stream);
}

}  // extern "C"
