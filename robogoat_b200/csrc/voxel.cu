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
#include "rc_common.cuh"

#include <atomic>
#include <mutex>

namespace {

constexpr int kThreads = 256;
constexpr int kPointsPerLane = 4;
constexpr int kPointsPerWarp = 32 * kPointsPerLane;            // 128
constexpr int kPointsPerBlock = kThreads * kPointsPerLane;     // 1024
constexpr size_t kResidentBytes = 96u << 20;   // accumulators up to this size are treated as L2-resident (one pass)
constexpr long long kProbeMinPoints = 1ll << 20;  // below this the order probe is not worth its launch
constexpr int kAutoMeanPasses = 6;             // slab passes of the two-phase mean scatter on larger grids
constexpr double kSlabPassBytes = 448.0 * 1048576.0;          // accumulator bytes per slab pass of rc_voxel_scatter_ids
constexpr size_t kSmallGridBytes = 64u << 20;                  // grids up to this size are cleared by voxel_zero_kernel

struct VoxelGeom {
    float minx, miny, minz, vs;
    int gx, gy, gz;
    float fgx, fgy, fgz;
};

// flat voxel id, or -1 for a dropped point (NaN and infinities fail the range test)
__device__ __forceinline__ long long voxel_id(float x, float y, float z, const VoxelGeom& g) {
    const float fx = floorf(__fdiv_rn(__fsub_rn(x, g.minx), g.vs));
    const float fy = floorf(__fdiv_rn(__fsub_rn(y, g.miny), g.vs));
    const float fz = floorf(__fdiv_rn(__fsub_rn(z, g.minz), g.vs));
    const bool in = (fx >= 0.0f) && (fx < g.fgx) && (fy >= 0.0f) && (fy < g.fgy) && (fz >= 0.0f) && (fz < g.fgz);
    if (!in) return -1;
    return (static_cast<long long>(fz) * g.gy + static_cast<long long>(fy)) * g.gx + static_cast<long long>(fx);
}

__device__ __forceinline__ void red_add_v4(float* addr, float4 v) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};"
                 :: "l"(addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
__device__ __forceinline__ void red_add_v2(float* addr, float2 v) {
    asm volatile("red.global.add.v2.f32 [%0], {%1, %2};" :: "l"(addr), "f"(v.x), "f"(v.y) : "memory");
}

// ordered-integer image of a float: larger float <=> larger signed int
__device__ __forceinline__ int float_ordered(float f) {
    const int i = __float_as_int(f);
    return (i >= 0) ? i : (i ^ 0x7fffffff);
}

enum : int { kCount = 0, kOccupancy = 1, kMean = 2, kMax = 3, kOccupancyU8 = 4 };

// The xyz of a warp's 128-point tile: point i of a lane is (base + i*32 + lane).
// Fast tiles (full, 16-byte aligned) are fetched with three coalesced 16-byte loads per lane
// (tile_issue), issued one tile ahead of their use, and transposed through the warp's slice of
// shared memory (tile_unpack); other tiles are read with scalar loads (tile_load_slow).
__device__ __forceinline__ void tile_issue(const float* __restrict__ pts, long long base, int lane, float4 (&v)[3]) {
    const float4* src = reinterpret_cast<const float4*>(pts + base * 3);
#pragma unroll
    for (int k = 0; k < 3; ++k) v[k] = __ldcs(src + k * 32 + lane);
}
__device__ __forceinline__ void tile_unpack(const float4 (&v)[3], float* s_warp, int lane,
                                            float (&x)[kPointsPerLane], float (&y)[kPointsPerLane],
                                            float (&z)[kPointsPerLane]) {
    float4* dst = reinterpret_cast<float4*>(s_warp);
#pragma unroll
    for (int k = 0; k < 3; ++k) dst[k * 32 + lane] = v[k];
    __syncwarp();
#pragma unroll
    for (int i = 0; i < kPointsPerLane; ++i) {
        const float* q = s_warp + (i * 32 + lane) * 3;  // stride of three words: conflict free
        x[i] = q[0]; y[i] = q[1]; z[i] = q[2];
    }
    __syncwarp();
}
__device__ __forceinline__ void tile_load_slow(const float* __restrict__ pts, long long base, long long N, int lane,
                                               float (&x)[kPointsPerLane], float (&y)[kPointsPerLane],
                                               float (&z)[kPointsPerLane]) {
#pragma unroll
    for (int i = 0; i < kPointsPerLane; ++i) {
        const long long pi = base + i * 32 + lane;
        if (pi < N) {
            x[i] = __ldg(pts + pi * 3 + 0);
            y[i] = __ldg(pts + pi * 3 + 1);
            z[i] = __ldg(pts + pi * 3 + 2);
        } else {
            x[i] = y[i] = z[i] = __int_as_float(0x7fc00000);  // NaN: dropped
        }
    }
}

// Programmatic dependent launch (sm_90+): a kernel launched with the programmatic-serialisation
// attribute may start while its predecessor in the stream is still running; it must execute
// grid_dependency_wait() before touching memory the predecessor writes.  Launched normally, the
// wait returns at once.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dependency_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Zero-fill for small grids (latency regime): lets the scatter kernel that follows be scheduled
// right away, so that its point loads and voxel-id arithmetic overlap this fill.
__global__ void __launch_bounds__(kThreads) voxel_zero_kernel(unsigned char* __restrict__ p, long long bytes) {
    grid_dependency_release();
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
constexpr int kProbeTiles = 256;
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

template <int MODE>
__device__ __forceinline__ void scatter_one(int id, long long pi, const float* __restrict__ feats, void* grid_v,
                                            int* __restrict__ counts, int F) {
    if (MODE == kCount) {
        atomicAdd(static_cast<int*>(grid_v) + id, 1);
    } else if (MODE == kOccupancy) {
        static_cast<int*>(grid_v)[id] = 1;
    } else {
        const float* f = feats + pi * F;
        float* o = static_cast<float*>(grid_v) + static_cast<long long>(id) * F;
        if ((F & 3) == 0) {
            for (int c = 0; c < F; c += 4) red_add_v4(o + c, __ldcs(reinterpret_cast<const float4*>(f + c)));
        } else if ((F & 1) == 0) {
            for (int c = 0; c < F; c += 2) red_add_v2(o + c, __ldcs(reinterpret_cast<const float2*>(f + c)));
        } else {
            for (int c = 0; c < F; ++c) atomicAdd(o + c, __ldg(f + c));
        }
        atomicAdd(counts + id, 1);
    }
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
voxel_normalize_wide_kernel(float* __restrict__ grid, const int* __restrict__ counts, long long v0, long long v1, int F) {
    __shared__ int s_vox[kThreads / 32][256];
    __shared__ int s_cnt[kThreads / 32][256];
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

// mean pass 2, one voxel per thread: ragged ends of a range and unaligned buffers
__global__ void __launch_bounds__(kThreads)
voxel_normalize_scalar_kernel(float* __restrict__ grid, const int* __restrict__ counts, long long v0, long long v1, int F) {
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

// ---------------------------------------------------------------- partition by owning part (point exchange)
//
// A stable counting partition in three launches.  Every CTA owns a contiguous run of 1024-point
// chunks.  Launch 1 (MOVE = false) counts the in-grid points per CTA and part; launch 2 turns each
// part's column of that table into exclusive prefixes over the CTAs (one CTA per part); launch 3
// (MOVE = true) walks the same chunks again - the count pass leaves every point's voxel id in the
// scratch, so the coordinates are not read twice -, sorts each chunk by part in shared memory and writes
// the sorted chunk out, so that every part receives runs of consecutive records: full-width stores
// whether the destination is local memory or a peer's.  Ranks inside a warp come from
// __match_any_sync and warps are prefixed in order, so input order is kept inside a part and the
// result does not depend on scheduling.
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

// voxel_id for grids of fewer than 2^31 voxels: the same float arithmetic, 32-bit index arithmetic
__device__ __forceinline__ int voxel_id32(float x, float y, float z, const VoxelGeom& g) {
    const float fx = floorf(__fdiv_rn(__fsub_rn(x, g.minx), g.vs));
    const float fy = floorf(__fdiv_rn(__fsub_rn(y, g.miny), g.vs));
    const float fz = floorf(__fdiv_rn(__fsub_rn(z, g.minz), g.vs));
    const bool in = (fx >= 0.0f) && (fx < g.fgx) && (fy >= 0.0f) && (fy < g.fgy) && (fz >= 0.0f) && (fz < g.fgz);
    if (!in) return -1;
    return (static_cast<int>(fz) * g.gy + static_cast<int>(fy)) * g.gx + static_cast<int>(fx);
}

// Bulk asynchronous copy shared -> global (the TMA engine moves a whole run of sorted records with one
// request, to local or peer memory alike).  Both addresses 16-byte aligned, size a multiple of 16 bytes.
__device__ __forceinline__ void bulk_store(void* dst_global, const void* src_shared, unsigned int bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                 :: "l"(__cvta_generic_to_global(dst_global)),
                    "r"(static_cast<unsigned int>(__cvta_generic_to_shared(src_shared))), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read_all_but_one() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_shared() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

template <bool MOVE, bool BULK>
__global__ void __launch_bounds__(kThreads, 5)
voxel_part_kernel(const float* __restrict__ pts, const float* __restrict__ feats, long long N, int F, VoxelGeom g,
                  bool pts_aligned, bool vec4, PartRule rule, long long chunks_per_cta, int* __restrict__ table,
                  int* __restrict__ ids_tmp, const long long* __restrict__ part_counts,
                  const __grid_constant__ PartDest dest) {
    __shared__ __align__(16) float s_xyz[MOVE ? 1 : kThreads / 32][MOVE ? 4 : kPointsPerWarp * 3];
    // count pass: per-warp totals.  move pass: this chunk's per-warp counts, turned by warp 0 into the
    // first slot of every (warp, part) in the sorted chunk
    __shared__ int s_wcnt[kThreads / 32][kMaxParts];
    __shared__ long long s_cur[MOVE ? kMaxParts : 1];        // next slot of each part in its destination
    __shared__ int* s_adj_ids[MOVE ? kMaxParts : 1];         // destination of sorted slot j of part p is s_adj_*[p] + j
    __shared__ float* s_adj_feats[MOVE ? kMaxParts : 1];
    __shared__ int s_total;
    __shared__ int s_sid[MOVE ? kChunk : 1];                 // the chunk's voxel ids, sorted by part
    __shared__ unsigned short s_meta[MOVE ? kChunk : 1];     // (index in chunk << 6) | part
    // feature rows of the sorted chunk, staged for the bulk stores; two buffers so that a chunk is staged
    // while the previous one is still being read by the copy engine
    __shared__ __align__(16) float4 s_feat[BULK ? 2 : 1][BULK ? kChunk : 1];
    constexpr bool bulk = MOVE && BULK;                      // callers pass BULK only together with vec4
    float* pend_dst[2] = {nullptr, nullptr};                 // warp 0: the runs of the previous chunk, not yet issued
    int pend_src[2] = {0, 0}, pend_cnt[2] = {0, 0}, pend_buf = 0;
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
        if (bulk && warp == 0) {
            // the previous chunk's feature rows are staged (its threads fenced before the barrier): one bulk
            // store per part and lane
#pragma unroll
            for (int h = 0; h < 2; ++h)
                if (pend_cnt[h] > 0) bulk_store(pend_dst[h], &s_feat[pend_buf][pend_src[h]], static_cast<unsigned int>(pend_cnt[h]) * 16u);
            bulk_commit();
        }
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
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int p = lane + 32 * h;
                if (p < P) {
                    const long long first = s_cur[p] - lstart[h];
                    s_adj_ids[p] = dest.ids[p] + first;
                    s_adj_feats[p] = (dest.feats[p] != nullptr) ? dest.feats[p] + first * F : nullptr;
                    pend_dst[h] = bulk ? dest.feats[p] + s_cur[p] * 4 : nullptr;
                    pend_src[h] = lstart[h];
                    pend_cnt[h] = tot[h];
                    s_cur[p] += tot[h];
                } else {
                    pend_cnt[h] = 0;
                }
            }
            pend_buf = chunk & 1;
            if (bulk) bulk_wait_read_all_but_one();   // the buffer this chunk stages into was read two chunks ago
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
                    if (bulk) s_feat[chunk & 1][j] = f4[m];
                    else reinterpret_cast<float4*>(s_adj_feats[p])[j] = f4[m];
                }
            }
            if (bulk) fence_async_shared();   // staged rows become visible to the copy engine; issued after the next barrier
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
        // no barrier here: the next chunk's first barrier comes before anything above is overwritten
    }
    if (MOVE && bulk) {
        __syncthreads();
        if (warp == 0) {
#pragma unroll
            for (int h = 0; h < 2; ++h)
                if (pend_cnt[h] > 0) bulk_store(pend_dst[h], &s_feat[pend_buf][pend_src[h]], static_cast<unsigned int>(pend_cnt[h]) * 16u);
            bulk_commit();
            bulk_wait_all();                  // shared memory must outlive the copies
        }
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
void launch_scatter_runs(unsigned int nb, cudaStream_t st, const int* ids, const float* feats, void* grid0, int* counts0,
                         int F, bool vec4, const RunTable& rt, int id_lo, unsigned int span) {
    voxel_scatter_runs_kernel<MODE><<<nb, kThreads, 0, st>>>(ids, feats, grid0, counts0, F, vec4, rt, id_lo, span);
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
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // [voxel_begin, head) and [body_end, voxel_end) go voxel by voxel; the body, whose count
    // pointer is 16-byte aligned and whose length is a multiple of four, goes four per thread
    long long head = voxel_begin;
    while (head < voxel_end && !rc::aligned_to(counts + head, 16)) ++head;
    const long long body_end = head + ((voxel_end - head) & ~3ll);
    auto scalar = [&](long long a, long long b) {
        if (b > a) {
            const long long blocks = (b - a + kThreads - 1) / kThreads;
            voxel_normalize_scalar_kernel<<<static_cast<unsigned int>(blocks), kThreads, 0, st>>>(grid, counts, a, b, F);
        }
    };
    if ((voxel_end - voxel_begin + kThreads - 1) / kThreads >= (1ll << 31)) return RC_ERR_TOO_LARGE;
    scalar(voxel_begin, head);
    if (body_end > head) {
        long long blocks = (((body_end - head) + 255) / 256 + kThreads / 32 - 1) / (kThreads / 32);
        const long long cap = 16ll * rc::sm_count(device);
        if (blocks > cap) blocks = cap;
        const unsigned int nb = static_cast<unsigned int>(blocks);
        if ((F & 3) == 0 && rc::aligned_to(grid, 16))
            voxel_normalize_wide_kernel<true><<<nb, kThreads, 0, st>>>(grid, counts, head, body_end, F);
        else
            voxel_normalize_wide_kernel<false><<<nb, kThreads, 0, st>>>(grid, counts, head, body_end, F);
    }
    scalar(body_end, voxel_end);
    return rc::check_launch();
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
    if (acc_bytes <= static_cast<double>(kResidentBytes)) return 0;  // L2-resident accumulators: one pass
    if (mode == RC_VOXEL_COUNT) return (N >= kProbeMinPoints) ? 16 : 0;     // the order probe's flag
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
                            const int64_t* dest_start, const int64_t* part_counts_device, const void* scratch,
                            uint64_t scratch_bytes, int device, void* stream) {
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
    // bulk (TMA) stores of the feature runs pay off over NVLink, per-thread stores in local memory
    const int bulk_opt = rc::g_part_bulk_store.load(std::memory_order_relaxed);
    bool bulk = vec4 && bulk_opt == 2;
    if (vec4 && bulk_opt == 1) {
        const float* seen = nullptr;
        for (int p = 0; p < rule.P && !bulk; ++p) {
            if (dest.feats[p] == seen) continue;
            seen = dest.feats[p];
            cudaPointerAttributes attr{};
            if (cudaPointerGetAttributes(&attr, seen) != cudaSuccess) { cudaGetLastError(); continue; }
            bulk = attr.type == cudaMemoryTypeDevice && attr.device != device;
        }
    }
    int* table = const_cast<int*>(static_cast<const int*>(scratch));
    int* ids_tmp = reinterpret_cast<int*>(const_cast<unsigned char*>(static_cast<const unsigned char*>(scratch)) +
                                          partition_table_bytes(blocks, rule.P));
    const unsigned int nb = static_cast<unsigned int>(blocks);
    const float* f_in = move_feats ? features : nullptr;
    const long long* pc_dev = reinterpret_cast<const long long*>(part_counts_device);
    if (bulk)
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
                                   part_counts, scratch, scratch_bytes, device, stream);
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
        for (int ps = 0; ps < n_passes; ++ps) {
            RunTable rt{};
            auto flush = [&]() {
                if (rt.n == 0) return;
                long long nb = rt.first_block[rt.n];
                if (nb > cap) nb = cap;
                const unsigned int blocks = static_cast<unsigned int>(nb);
                const int lo = static_cast<int>(id_begin);
                const unsigned int span = static_cast<unsigned int>(nvox);
                if (mode == RC_VOXEL_MEAN) launch_scatter_runs<kMean>(blocks, st, ids, features, grid0, counts0, F, vec4, rt, lo, span);
                else if (mode == RC_VOXEL_COUNT) launch_scatter_runs<kCount>(blocks, st, ids, features, grid0, counts0, F, false, rt, lo, span);
                else launch_scatter_runs<kOccupancy>(blocks, st, ids, features, grid0, counts0, F, false, rt, lo, span);
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
