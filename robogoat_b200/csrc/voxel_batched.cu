// Batched voxel grids in one launch: [B, N, 3] clouds -> [B, D, H, W(, F)] float grids, and per-item
// bounding boxes.  This is the older operator surface of the reference
// (robocache/kernels/cutlass/point_cloud_voxelization.h:59-157, kernels in point_cloud_voxelization.cu):
// float occupancy (0/1), float density (points per voxel), feature mean, feature max, and compute_point_cloud_bounds.
//
// The batch is one flat list of B*N points; the item index is folded into the voxel id
// (id = b * D*H*W + vz*H*W + vy*W + vx), so a single launch bins every item into its slice of one batch
// grid that was cleared with one fill.  The cell arithmetic is the single-cloud operator's (IEEE fp32
// subtraction, division, floor; out-of-grid points dropped) - the same rule as the reference's
// point_to_voxel_idx (point_cloud_voxelization.cu:23-39).
#include "voxel_common.cuh"

namespace {

using namespace rc::vox;

enum : int { kBatchOccupancy = 0, kBatchDensity = 1, kBatchMean = 2, kBatchMax = 3 };

__device__ __forceinline__ void red_add_f32(float* addr, float v) {
    asm volatile("red.global.add.f32 [%0], %1;" :: "l"(addr), "f"(v) : "memory");
}

// A warp takes 128 consecutive points of the flat list (a tile may straddle items).
template <int MODE>
__global__ void __launch_bounds__(kThreads)
voxel_batched_kernel(const float* __restrict__ pts, const float* __restrict__ feats, float* __restrict__ grid,
                     int* __restrict__ counts, long long total, long long N, int F, VoxelGeom g, long long V,
                     bool pts_aligned) {
    __shared__ __align__(16) float s_xyz[kThreads / 32][kPointsPerWarp * 3];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const long long ntiles = (total + kPointsPerWarp - 1) / kPointsPerWarp;
    const long long warps_total = static_cast<long long>(gridDim.x) * (kThreads / 32);
    for (long long tile = static_cast<long long>(blockIdx.x) * (kThreads / 32) + warp; tile < ntiles; tile += warps_total) {
        const long long base = tile * kPointsPerWarp;
        float x[kPointsPerLane], y[kPointsPerLane], z[kPointsPerLane];
        if (pts_aligned && base + kPointsPerWarp <= total) {
            float4 cur[3];
            tile_issue(pts, base, lane, cur);
            tile_unpack(cur, s_xyz[warp], lane, x, y, z);
        } else {
            tile_load_slow(pts, base, total, lane, x, y, z);
        }
        const long long b0 = base / N;                       // item of the tile's first point
#pragma unroll
        for (int i = 0; i < kPointsPerLane; ++i) {
            const long long pi = base + i * 32 + lane;
            const long long id = voxel_id(x[i], y[i], z[i], g);
            if (id < 0 || pi >= total) continue;
            long long b = b0;
            if (N >= kPointsPerWarp) {                       // at most one item boundary inside the tile
                if (pi - b0 * N >= N) ++b;
            } else {
                b = pi / N;
            }
            const long long cell = b * V + id;
            if (MODE == kBatchOccupancy) {
                grid[cell] = 1.0f;                           // every writer stores the same value
            } else if (MODE == kBatchDensity) {
                red_add_f32(grid + cell, 1.0f);              // exact below 2^24 points per voxel
            } else if (MODE == kBatchMax) {
                // the reference's kernel takes fmaxf against a grid that starts at zero (point_cloud_voxelization.cu:
                // 139-195): the result is max(0, max of the features); positive floats order like their bit patterns
                const float* f = feats + pi * F;
                int* o = reinterpret_cast<int*>(grid) + cell * F;
                for (int c = 0; c < F; ++c) {
                    const float v = __ldg(f + c);
                    if (v > 0.0f) atomicMax(o + c, __float_as_int(v));
                }
            } else {
                const float* f = feats + pi * F;
                float* o = grid + cell * F;
                if ((F & 3) == 0) {
                    for (int c = 0; c < F; c += 4) red_add_v4(o + c, __ldcs(reinterpret_cast<const float4*>(f + c)));
                } else if ((F & 1) == 0) {
                    for (int c = 0; c < F; c += 2) red_add_v2(o + c, __ldcs(reinterpret_cast<const float2*>(f + c)));
                } else {
                    for (int c = 0; c < F; ++c) red_add_f32(o + c, __ldg(f + c));
                }
                atomicAdd(counts + cell, 1);
            }
        }
    }
}

// One CTA per item: minimum and maximum of every coordinate, starting from +-1e10 as the reference does
// (point_cloud_voxelization.cu:386-449); NaN coordinates are ignored by fminf / fmaxf.
__global__ void __launch_bounds__(kThreads)
voxel_bounds_kernel(const float* __restrict__ pts, float* __restrict__ lo, float* __restrict__ hi, long long N) {
    __shared__ float s_lo[kThreads / 32][3], s_hi[kThreads / 32][3];
    const long long b = blockIdx.x;
    const float* p = pts + b * N * 3;
    float mn[3] = {1e10f, 1e10f, 1e10f}, mx[3] = {-1e10f, -1e10f, -1e10f};
    for (long long i = threadIdx.x; i < N; i += kThreads) {
#pragma unroll
        for (int a = 0; a < 3; ++a) {
            const float v = __ldg(p + i * 3 + a);
            mn[a] = fminf(mn[a], v);
            mx[a] = fmaxf(mx[a], v);
        }
    }
#pragma unroll
    for (int a = 0; a < 3; ++a) {
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            mn[a] = fminf(mn[a], __shfl_xor_sync(0xffffffffu, mn[a], off));
            mx[a] = fmaxf(mx[a], __shfl_xor_sync(0xffffffffu, mx[a], off));
        }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) {
#pragma unroll
        for (int a = 0; a < 3; ++a) { s_lo[warp][a] = mn[a]; s_hi[warp][a] = mx[a]; }
    }
    __syncthreads();
    if (threadIdx.x < 3) {
        float m = s_lo[0][threadIdx.x], M = s_hi[0][threadIdx.x];
        for (int w = 1; w < kThreads / 32; ++w) { m = fminf(m, s_lo[w][threadIdx.x]); M = fmaxf(M, s_hi[w][threadIdx.x]); }
        lo[b * 3 + threadIdx.x] = m;
        hi[b * 3 + threadIdx.x] = M;
    }
}

}  // namespace

extern "C" {

int rc_voxelize_batched(const float* points, const float* features, float* grid, int32_t* counts, int64_t B, int64_t N,
                        int32_t F, const float origin_host[3], float voxel_size, const int32_t dhw_host[3], int mode,
                        uint32_t flags, int device, void* stream) {
    if (mode != RC_BATCHED_OCCUPANCY && mode != RC_BATCHED_DENSITY && mode != RC_BATCHED_FEATURE_MEAN &&
        mode != RC_BATCHED_FEATURE_MAX)
        return RC_ERR_BAD_MODE;
    if (origin_host == nullptr || dhw_host == nullptr) return RC_ERR_NULL_POINTER;
    if (B < 0 || N < 0 || F < 0) return RC_ERR_BAD_SHAPE;
    if (!(voxel_size > 0.0f) || !(voxel_size <= 3.0e38f)) return RC_ERR_BAD_VALUE;
    const bool mean = (mode == RC_BATCHED_FEATURE_MEAN);
    const bool feat = mean || mode == RC_BATCHED_FEATURE_MAX;
    VoxelGeom g;
    g.minx = origin_host[0]; g.miny = origin_host[1]; g.minz = origin_host[2];
    g.vs = voxel_size;
    g.gz = dhw_host[0]; g.gy = dhw_host[1]; g.gx = dhw_host[2];            // depth = z, height = y, width = x
    if (g.gx < 0 || g.gy < 0 || g.gz < 0) return RC_ERR_BAD_SHAPE;
    if (g.gx >= (1 << 24) || g.gy >= (1 << 24) || g.gz >= (1 << 24)) return RC_ERR_TOO_LARGE;
    g.fgx = static_cast<float>(g.gx); g.fgy = static_cast<float>(g.gy); g.fgz = static_cast<float>(g.gz);
    g.inv_vs = host_reciprocal(voxel_size);
    const double cells_d = static_cast<double>(g.gx) * g.gy * g.gz * static_cast<double>(B) * (feat ? (F > 0 ? F : 1) : 1);
    if (cells_d >= 1099511627776.0 || static_cast<double>(B) * static_cast<double>(N) >= 4.0e18) return RC_ERR_TOO_LARGE;
    const long long V = static_cast<long long>(g.gx) * g.gy * g.gz;
    const long long cells = V * B * (feat ? F : 1);
    if (cells > 0 && grid == nullptr) return RC_ERR_NULL_POINTER;
    if (mean && V * B > 0 && counts == nullptr) return RC_ERR_NULL_POINTER;
    if (feat && B * N > 0 && F > 0 && features == nullptr) return RC_ERR_BAD_MODE;
    if (B * N > 0 && points == nullptr) return RC_ERR_NULL_POINTER;
    if (!rc::aligned_to(points, 4) || !rc::aligned_to(features, 4) || !rc::aligned_to(grid, 4) || !rc::aligned_to(counts, 4))
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
    if (flags & RC_VOXEL_ZERO_INIT) {
        if (cells > 0) RC_CUDA_TRY(cudaMemsetAsync(grid, 0, static_cast<size_t>(cells) * 4, st));
        if (mean && V * B > 0) RC_CUDA_TRY(cudaMemsetAsync(counts, 0, static_cast<size_t>(V * B) * 4, st));
    }
    const long long total = B * N;
    if (total > 0 && V > 0 && !(feat && F == 0)) {
        long long blocks = (total + kPointsPerBlock - 1) / kPointsPerBlock;
        const long long cap = 16ll * rc::sm_count(device);
        if (blocks > cap) blocks = cap;
        const unsigned int nb = static_cast<unsigned int>(blocks);
        const bool aligned = rc::aligned_to(points, 16);
        if (mode == RC_BATCHED_OCCUPANCY)
            voxel_batched_kernel<kBatchOccupancy><<<nb, kThreads, 0, st>>>(points, features, grid, counts, total, N, F, g, V, aligned);
        else if (mode == RC_BATCHED_DENSITY)
            voxel_batched_kernel<kBatchDensity><<<nb, kThreads, 0, st>>>(points, features, grid, counts, total, N, F, g, V, aligned);
        else if (mode == RC_BATCHED_FEATURE_MAX)
            voxel_batched_kernel<kBatchMax><<<nb, kThreads, 0, st>>>(points, features, grid, counts, total, N, F, g, V, aligned);
        else
            voxel_batched_kernel<kBatchMean><<<nb, kThreads, 0, st>>>(points, features, grid, counts, total, N, F, g, V, aligned);
    }
    const int rc_launch = rc::check_launch();
    if (rc_launch != RC_OK) return rc_launch;
    if (mean && !(flags & RC_VOXEL_NO_NORMALIZE) && V * B > 0 && F > 0)
        return rc_voxel_normalize(grid, counts, 0, V * B, F, device, stream);
    return RC_OK;
}

int rc_point_cloud_bounds(const float* points, float* min_bounds, float* max_bounds, int64_t B, int64_t N, int device,
                          void* stream) {
    if (B < 0 || N < 0) return RC_ERR_BAD_SHAPE;
    if (B == 0) return RC_OK;
    if (B >= (1ll << 31)) return RC_ERR_TOO_LARGE;
    if (min_bounds == nullptr || max_bounds == nullptr || (N > 0 && points == nullptr)) return RC_ERR_NULL_POINTER;
    if (!rc::aligned_to(points, 4) || !rc::aligned_to(min_bounds, 4) || !rc::aligned_to(max_bounds, 4)) return RC_ERR_BAD_ALIGNMENT;
    rc::DeviceScope scope(device);
    if (scope.status() != RC_OK) return scope.status();
    voxel_bounds_kernel<<<static_cast<unsigned int>(B), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(points, min_bounds, max_bounds, N);
    return rc::check_launch();
}

}  // extern "C"
