// Truncated signed distance grids from batched point clouds: points [B,N,3] (+ optional unit normals [B,N,3])
// -> tsdf fp32 [B,D,H,W] in [-1,1] and weight fp32 [B,D,H,W] (points within the truncation distance of the
// voxel centre).  This is voxelize_tsdf of the reference's older operator surface
// (robocache/kernels/cutlass/point_cloud_voxelization.h:146-173, kernel point_cloud_voxelization.cu:278-376).
//
// The reference keeps, per voxel, the smallest |distance| / truncation over the points whose distance to the voxel
// centre is below the truncation distance, with a compare-and-swap loop that gives the result the sign of whichever
// point reached the voxel first - so with normals its sign depends on the order the threads ran in.  Here the sign
// is that of the CLOSEST point (ties: outside wins), which is what the reference returns whenever its result does
// not depend on that order (no normals, or all contributing points on one side).  That makes the update a plain
// integer minimum: a distance in [0,1] has a bit pattern below 2^30, so key = (bits << 1) | inside orders first by
// distance and then by side, and one atomicMin per (point, voxel) replaces the compare-and-swap loop.  A last pass
// turns keys into floats (empty voxels: 0, as in the reference, whose grids start at zero).
//
// A warp takes 32 points; for each of them in turn its lanes spread over the (y, x) cells of the voxel neighbourhood
// (x fastest, so the atomics of one step fall on consecutive addresses) and walk their columns in z.
#include "voxel_common.cuh"

namespace {

using namespace rc::vox;

constexpr unsigned int kTsdfEmpty = 0xffffffffu;

struct TsdfGeom {
    float ox, oy, oz, vs, trunc, inv_trunc;
    int gx, gy, gz, reach;          // reach: voxels searched either side of the point's own voxel
};

__device__ __forceinline__ void red_add_one(float* addr) {
    asm volatile("red.global.add.f32 [%0], %1;" :: "l"(addr), "f"(1.0f) : "memory");
}

// Range of cells [lo, hi] on one axis within `reach` of the cell that holds p, clipped to the grid; false if empty.
__device__ __forceinline__ bool axis_range(float p, float o, float vs, int reach, int dim, int& lo, int& hi) {
    const float c = floorf((p - o) / vs);
    const float flo = fmaxf(c - static_cast<float>(reach), 0.0f);
    const float fhi = fminf(c + static_cast<float>(reach), static_cast<float>(dim - 1));
    if (!(flo <= fhi)) return false;            // also drops NaN
    lo = static_cast<int>(flo);
    hi = static_cast<int>(fhi);
    return true;
}

__global__ void __launch_bounds__(kThreads)
voxel_tsdf_kernel(const float* __restrict__ pts, const float* __restrict__ normals, unsigned int* __restrict__ keys,
                  float* __restrict__ weights, long long total, long long N, TsdfGeom g, long long V) {
    const int lane = threadIdx.x & 31;
    const long long warp = (static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x) >> 5;
    const long long warps_total = (static_cast<long long>(gridDim.x) * kThreads) >> 5;
    const long long plane = static_cast<long long>(g.gx) * g.gy;
    for (long long base = warp * 32; base < total; base += warps_total * 32) {
        const long long mine = base + lane;
        float px = 0.f, py = 0.f, pz = 0.f, nx = 0.f, ny = 0.f, nz = 0.f;
        if (mine < total) {
            px = __ldg(pts + mine * 3 + 0); py = __ldg(pts + mine * 3 + 1); pz = __ldg(pts + mine * 3 + 2);
            if (normals != nullptr) {
                nx = __ldg(normals + mine * 3 + 0); ny = __ldg(normals + mine * 3 + 1); nz = __ldg(normals + mine * 3 + 2);
            }
        }
        const int npts = static_cast<int>(min(32ll, total - base));
        for (int j = 0; j < npts; ++j) {
            const float x = __shfl_sync(0xffffffffu, px, j), y = __shfl_sync(0xffffffffu, py, j), z = __shfl_sync(0xffffffffu, pz, j);
            const float ax = __shfl_sync(0xffffffffu, nx, j), ay = __shfl_sync(0xffffffffu, ny, j), az = __shfl_sync(0xffffffffu, nz, j);
            int x0, x1, y0, y1, z0, z1;
            if (!axis_range(x, g.ox, g.vs, g.reach, g.gx, x0, x1)) continue;     // uniform across the warp
            if (!axis_range(y, g.oy, g.vs, g.reach, g.gy, y0, y1)) continue;
            if (!axis_range(z, g.oz, g.vs, g.reach, g.gz, z0, z1)) continue;
            const unsigned int wx = x1 - x0 + 1, wy = y1 - y0 + 1;
            const unsigned int nplane = wx * wy;                                   // <= 1025^2
            const long long item = ((base + j) / N) * V;
            // lanes over the (y, x) cells of the neighbourhood, z as the inner loop: the cell's x/y offsets, their
            // squares and the x/y part of the normal's dot product are computed once per column.  c / wx comes from one
            // reciprocal per point: floor(c * ceil(2^32 / wx) / 2^32) is exact while c * wx < 2^32, and c < 1025^2,
            // wx <= 1025 (wx = 1 has no 32-bit reciprocal).
            const unsigned int mx = static_cast<unsigned int>((0x100000000ull + wx - 1) / wx);
            for (unsigned int c = lane; c < nplane; c += 32) {
                const unsigned int r = (wx == 1) ? c : __umulhi(c, mx);
                const int vx = x0 + static_cast<int>(c - r * wx);
                const int vy = y0 + static_cast<int>(r);
                // voxel centre and distance: single fp32 operations in this order (no contraction)
                const float dx = (g.ox + (static_cast<float>(vx) + 0.5f) * g.vs) - x;
                const float dy = (g.oy + (static_cast<float>(vy) + 0.5f) * g.vs) - y;
                const float dxy2 = dx * dx + dy * dy;
                // rounded addition and square root are monotonic: a column whose x/y offset alone reaches the
                // truncation distance has no cell inside it
                if (!(sqrtf(dxy2) < g.trunc)) continue;
                const float dotxy = ax * dx + ay * dy;
                long long cell = item + static_cast<long long>(z0) * plane + static_cast<long long>(vy) * g.gx + vx;
                for (int vz = z0; vz <= z1; ++vz, cell += plane) {
                    const float dz = (g.oz + (static_cast<float>(vz) + 0.5f) * g.vs) - z;
                    const float dist = sqrtf(dxy2 + dz * dz);
                    if (!(dist < g.trunc)) continue;
                    unsigned int inside = 0u;
                    if (normals != nullptr && (dotxy + az * dz) > 0.0f) inside = 1u;
                    const float val = fminf(1.0f, dist * g.inv_trunc);
                    atomicMin(keys + cell, (__float_as_uint(val) << 1) | inside);
                    red_add_one(weights + cell);
                }
            }
        }
    }
}

__global__ void __launch_bounds__(kThreads)
voxel_tsdf_decode_kernel(unsigned int* __restrict__ keys, long long cells) {
    const long long stride = static_cast<long long>(gridDim.x) * kThreads;
    for (long long i = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x; i < cells; i += stride) {
        const unsigned int k = keys[i];
        float v = 0.0f;
        if (k != kTsdfEmpty) {
            v = __uint_as_float(k >> 1);
            if (k & 1u) v = -v;
        }
        keys[i] = __float_as_uint(v);
    }
}

}  // namespace

extern "C" int rc_voxelize_tsdf(const float* points, const float* normals, float* tsdf_grid, float* weight_grid, int64_t B,
                                int64_t N, const float origin_host[3], float voxel_size, const int32_t dhw_host[3],
                                float truncation_distance, int device, void* stream) {
    if (origin_host == nullptr || dhw_host == nullptr) return RC_ERR_NULL_POINTER;
    if (B < 0 || N < 0) return RC_ERR_BAD_SHAPE;
    if (!(voxel_size > 0.0f) || !(voxel_size <= 3.0e38f)) return RC_ERR_BAD_VALUE;
    if (!(truncation_distance > 0.0f) || !(truncation_distance <= 3.0e38f)) return RC_ERR_BAD_VALUE;
    TsdfGeom g;
    g.ox = origin_host[0]; g.oy = origin_host[1]; g.oz = origin_host[2];
    g.vs = voxel_size;
    g.trunc = truncation_distance;
    g.inv_trunc = 1.0f / truncation_distance;
    g.gz = dhw_host[0]; g.gy = dhw_host[1]; g.gx = dhw_host[2];            // depth = z, height = y, width = x
    if (g.gx < 0 || g.gy < 0 || g.gz < 0) return RC_ERR_BAD_SHAPE;
    if (g.gx >= (1 << 24) || g.gy >= (1 << 24) || g.gz >= (1 << 24)) return RC_ERR_TOO_LARGE;
    // the reference searches ceil(truncation / voxel) + 1 voxels either side (point_cloud_voxelization.cu:297); the
    // distance test decides membership, the reach only has to cover it
    const double reach_d = std::ceil(static_cast<double>(truncation_distance) / static_cast<double>(voxel_size)) + 1.0;
    if (!(reach_d <= 512.0)) return RC_ERR_TOO_LARGE;     // keeps a point's neighbourhood below 2^31 cells
    g.reach = static_cast<int>(reach_d);
    const double cells_d = static_cast<double>(g.gx) * g.gy * g.gz * static_cast<double>(B);
    if (cells_d >= 1099511627776.0 || static_cast<double>(B) * static_cast<double>(N) >= 4.0e18) return RC_ERR_TOO_LARGE;
    const long long V = static_cast<long long>(g.gx) * g.gy * g.gz;
    const long long cells = V * B;
    if (cells > 0 && (tsdf_grid == nullptr || weight_grid == nullptr)) return RC_ERR_NULL_POINTER;
    if (B * N > 0 && points == nullptr) return RC_ERR_NULL_POINTER;
    if (!rc::aligned_to(points, 4) || !rc::aligned_to(normals, 4) || !rc::aligned_to(tsdf_grid, 4) ||
        !rc::aligned_to(weight_grid, 4))
        return RC_ERR_BAD_ALIGNMENT;
    if (cells == 0) return RC_OK;
    rc::DeviceScope scope(device);
    if (scope.status() != RC_OK) return scope.status();
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    RC_CUDA_TRY(cudaMemsetAsync(tsdf_grid, 0xff, static_cast<size_t>(cells) * 4, st));
    RC_CUDA_TRY(cudaMemsetAsync(weight_grid, 0, static_cast<size_t>(cells) * 4, st));
    const long long total = B * N;
    const long long cap = 16ll * rc::sm_count(device);
    if (total > 0) {
        long long blocks = (total + kThreads - 1) / kThreads;
        if (blocks > cap) blocks = cap;
        voxel_tsdf_kernel<<<static_cast<unsigned int>(blocks), kThreads, 0, st>>>(
            points, normals, reinterpret_cast<unsigned int*>(tsdf_grid), weight_grid, total, N, g, V);
        const int rc_launch = rc::check_launch();
        if (rc_launch != RC_OK) return rc_launch;
    }
    long long blocks = (cells + kThreads * 4 - 1) / (kThreads * 4);
    if (blocks > cap) blocks = cap;
    voxel_tsdf_decode_kernel<<<static_cast<unsigned int>(blocks), kThreads, 0, st>>>(reinterpret_cast<unsigned int*>(tsdf_grid), cells);
    return rc::check_launch();
}
