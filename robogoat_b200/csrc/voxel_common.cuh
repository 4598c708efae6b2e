// Shared device code of the voxelisation kernels: grid geometry and the voxel id in IEEE fp32,
// the vector reductions, the 128-point tile loads and the per-point scatter.
#pragma once

#include "rc_common.cuh"

namespace rc {
namespace vox {


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
    float inv_vs;   // RN(1 / vs), computed on the host
};

// RN(1 / vs) for VoxelGeom::inv_vs; NaN when the reciprocal is not a normal float (its relative error would
// exceed 2^-24), which sends every point of axis_cell through the division
inline float host_reciprocal(float vs) {
    const float r = 1.0f / vs;
    return (r >= 1.1754944e-38f && r <= 3.4028235e38f) ? r : __builtin_nanf("");
}

// floor((p - lo) / vs) with the reference's rounding (one IEEE subtraction, one IEEE division,
// floor), at the price of a multiplication for almost every point.  t = a * RN(1/vs) and the
// exact quotient q = RN(a / vs) differ by less than |t| * 2^-22 (three roundings of 2^-24 each),
// so floor(t) == floor(q) whenever t is further than that from every integer, i.e. when its
// fractional part is closer to 0.5 than 0.5 - |t| * 2.5e-7.  Only the points that fail the test (a
// few in 10^4 at 512 cells per axis), quotients so small that the product could underflow (their
// fractional part rounds to 0 or 1), NaN and infinities take the division.
__device__ __forceinline__ float axis_cell(float p, float lo, float vs, float inv_vs) {
    const float a = __fsub_rn(p, lo);
    const float t = __fmul_rn(a, inv_vs);
    float f = floorf(t);
    const float off = fabsf(__fsub_rn(__fsub_rn(t, f), 0.5f));          // |frac(t) - 0.5|, in [0, 0.5]
    if (!(off < __fmaf_rn(fabsf(t), -2.5e-7f, 0.5f))) f = floorf(__fdiv_rn(a, vs));
    return f;
}

// flat voxel id, or -1 for a dropped point (NaN and infinities fail the range test)
__device__ __forceinline__ long long voxel_id(float x, float y, float z, const VoxelGeom& g) {
    const float fx = axis_cell(x, g.minx, g.vs, g.inv_vs);
    const float fy = axis_cell(y, g.miny, g.vs, g.inv_vs);
    const float fz = axis_cell(z, g.minz, g.vs, g.inv_vs);
    const bool in = (fx >= 0.0f) && (fx < g.fgx) && (fy >= 0.0f) && (fy < g.fgy) && (fz >= 0.0f) && (fz < g.fgz);
    if (!in) return -1;
    return (static_cast<long long>(fz) * g.gy + static_cast<long long>(fy)) * g.gx + static_cast<long long>(fx);
}

// voxel_id for grids of fewer than 2^31 voxels: the same float arithmetic, 32-bit index arithmetic
__device__ __forceinline__ int voxel_id32(float x, float y, float z, const VoxelGeom& g) {
    const float fx = axis_cell(x, g.minx, g.vs, g.inv_vs);
    const float fy = axis_cell(y, g.miny, g.vs, g.inv_vs);
    const float fz = axis_cell(z, g.minz, g.vs, g.inv_vs);
    const bool in = (fx >= 0.0f) && (fx < g.fgx) && (fy >= 0.0f) && (fy < g.fgy) && (fz >= 0.0f) && (fz < g.fgz);
    if (!in) return -1;
    return (static_cast<int>(fz) * g.gy + static_cast<int>(fy)) * g.gx + static_cast<int>(fx);
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

// ---- mean mode by slab-ordered runs (voxel_runs.cu), used by rc_voxelize_ex for F = 4 on grids whose
// accumulators exceed L2.  `parts` slabs (at most kMeanRunsMaxParts); scratch of mean_runs_scratch_bytes(),
// 256-byte aligned; grid and features 16-byte aligned; V < 2^31; N <= 2^31 - 4096.  The grid and the counters
// must be clear; the grid holds feature sums afterwards.
constexpr int kMeanRunsMaxParts = 16;
constexpr int kMeanRunsParts = 16;
uint64_t mean_runs_scratch_bytes(long long N, long long V, int parts);
int mean_runs_launch(const float* points, const float* features, float* grid, int* counts, long long N,
                     const VoxelGeom& g, long long V, int parts, void* scratch, const int* gate, int gate_want,
                     int device, cudaStream_t st);

}  // namespace vox
}  // namespace rc
