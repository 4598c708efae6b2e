// Sparse reduction of partial voxel grids across GPUs (mean mode with four feature channels, and count mode).
//
// When a cloud puts many points into each occupied voxel, a rank's partial grid holds far fewer occupied voxels than
// the rank has points (the 2^26-point mixture: 4.8 M of 134 M voxels), so after binning its own points into a private
// full-size grid a rank needs to send every other rank only the occupied voxels of that rank's slab - 24 bytes per
// occupied voxel instead of 20 bytes per point, and nothing at all for empty space.  Two kernels:
//   voxel_sparse_send_kernel   walks the counter plane of the slabs other ranks own, and appends (voxel id, feature
//                              sums, count) of every occupied voxel to this rank's region of the owner's record list
//                              (collected per warp in shared memory, written as contiguous runs of plain stores,
//                              possibly into peer memory; slots from a counter in local memory);
//   voxel_sparse_merge_kernel  the owner adds the records it received to its own slab of its own partial grid.
// A one-warp kernel publishes the record counts to the owners.  Record lists have a fixed capacity per (source,
// owner) pair; records beyond it are dropped and reported through an overflow flag that the caller must check.
// No counterpart in the reference, whose multi-GPU test all-reduces dense grids (robocache/tests/test_multi_gpu.py:76).
#include "voxel_common.cuh"

namespace {

using namespace rc::vox;

constexpr int kSparseMaxPeers = 16;
constexpr int kSparseTile = 128;                // voxels a warp examines per step

struct SparseDests {
    long long begin[kSparseMaxPeers], end[kSparseMaxPeers];     // voxel ranges, one per destination
    long long tile0[kSparseMaxPeers + 1];                       // first 128-voxel tile of every range in the flat tile list
    int* ids[kSparseMaxPeers];
    float4* sums[kSparseMaxPeers];
    int* cnts[kSparseMaxPeers];
    int* nrec[kSparseMaxPeers];
    int n;
};

// A warp walks a contiguous run of 128-voxel tiles (four voxels per lane and step), collects the occupied voxels'
// records in its own piece of shared memory and, whenever more than kSparseFlush are waiting (or the destination
// changes), reserves their slots with ONE atomic on the destination's cursor and writes them out as three contiguous
// runs.  History of this kernel, 2^26-point mixture, 2 GPUs, 62 MB to send: every warp writing its handful of records
// straight to the peer 0.51 ms (each partial line is a packet of its own on NVLink, and the packet rate bounded it,
// not the bytes); records collected per CTA of 1024 voxels with two barriers per step 0.15-0.25 ms and issue-bound
// (220 instructions per warp and step); per warp, no barrier, tiles without an occupied voxel left after one vote:
// this form.
constexpr int kSparseFlush = 64;
constexpr int kSparseStage = kSparseFlush + kSparseTile;

__device__ __forceinline__ void sparse_flush(const SparseDests& d, int r, int fill, int* cursor, long long capacity,
                                             const int* s_ids, const float4* s_sums, const int* s_cnts, int lane) {
    int base = 0;
    if (lane == 0) base = atomicAdd(cursor + r, fill);
    base = __shfl_sync(0xffffffffu, base, 0);
    for (int i = lane; i < fill; i += 32) {
        const long long slot = static_cast<long long>(base) + i;
        if (slot < capacity) {
            d.ids[r][slot] = s_ids[i];
            if (d.sums[r] != nullptr) d.sums[r][slot] = s_sums[i];
            d.cnts[r][slot] = s_cnts[i];
        }
    }
    __syncwarp();                                                 // the staging arrays are free again
}

__global__ void __launch_bounds__(kThreads)
voxel_sparse_send_kernel(const float4* __restrict__ grid, const int* __restrict__ counts, SparseDests d, int* __restrict__ cursor,
                         long long capacity) {
    __shared__ __align__(16) float4 s_sums_all[kThreads / 32][kSparseStage];
    __shared__ int s_ids_all[kThreads / 32][kSparseStage];
    __shared__ int s_cnts_all[kThreads / 32][kSparseStage];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    float4* s_sums = s_sums_all[warp];
    int* s_ids = s_ids_all[warp];
    int* s_cnts = s_cnts_all[warp];
    const long long ntiles = d.tile0[d.n];
    const long long nwarps = static_cast<long long>(gridDim.x) * (kThreads / 32);
    const long long per = (ntiles + nwarps - 1) / nwarps;
    const long long t0 = (static_cast<long long>(blockIdx.x) * (kThreads / 32) + warp) * per;
    const long long t1 = (t0 + per < ntiles) ? t0 + per : ntiles;
    int fill = 0, fill_r = 0;                                     // staged records and their destination (warp-uniform)
    // the counters of the next tile are requested before this tile's are used
    int rn = 0;
    long long vn = 0;
    int cn[4] = {0, 0, 0, 0};
    auto fetch = [&](long long tile) {
        while (rn + 1 < d.n && tile >= d.tile0[rn + 1]) ++rn;
        vn = d.begin[rn] + (tile - d.tile0[rn]) * kSparseTile + lane * 4;
        cn[0] = cn[1] = cn[2] = cn[3] = 0;
        if (vn + 4 <= d.end[rn] && ((vn & 3) == 0)) {
            const int4 q = __ldcs(reinterpret_cast<const int4*>(counts + vn));
            cn[0] = q.x; cn[1] = q.y; cn[2] = q.z; cn[3] = q.w;
        } else {
#pragma unroll
            for (int k = 0; k < 4; ++k)
                if (vn + k < d.end[rn]) cn[k] = __ldcs(counts + vn + k);
        }
    };
    if (t0 < t1) fetch(t0);
    for (long long tile = t0; tile < t1; ++tile) {
        const int r = rn;
        const long long v0 = vn;
        const int c[4] = {cn[0], cn[1], cn[2], cn[3]};
        if (tile + 1 < t1) fetch(tile + 1);
        const int mine = (c[0] > 0) + (c[1] > 0) + (c[2] > 0) + (c[3] > 0);
        if (!__any_sync(0xffffffffu, mine)) continue;             // most tiles of a sparse grid hold no occupied voxel
        if (r != fill_r) {
            if (fill > 0) sparse_flush(d, fill_r, fill, cursor, capacity, s_ids, s_sums, s_cnts, lane);
            fill = 0;
            fill_r = r;
        }
        float4 sv[4] = {};
        if (grid != nullptr) {                                    // count mode has no feature sums
#pragma unroll
            for (int k = 0; k < 4; ++k)
                if (c[k] > 0) sv[k] = __ldcs(grid + v0 + k);      // in flight across the prefix sum
        }
        int incl = mine;                                          // inclusive prefix sum over the warp
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const int up = __shfl_up_sync(0xffffffffu, incl, off);
            if (lane >= off) incl += up;
        }
        const int total = __shfl_sync(0xffffffffu, incl, 31);
        int at = fill + (incl - mine);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            if (c[k] > 0) {
                s_ids[at] = static_cast<int>(v0 + k);
                s_sums[at] = sv[k];
                s_cnts[at] = c[k];
                ++at;
            }
        }
        __syncwarp();                                             // records staged
        fill += total;
        if (fill > kSparseFlush) {                                // the next step may add up to kSparseTile records
            sparse_flush(d, fill_r, fill, cursor, capacity, s_ids, s_sums, s_cnts, lane);
            fill = 0;
        }
    }
    if (fill > 0) sparse_flush(d, fill_r, fill, cursor, capacity, s_ids, s_sums, s_cnts, lane);
}

// The counts reach the owners after the records (stream order); a count above the capacity raises the local flag.
__global__ void voxel_sparse_publish_kernel(SparseDests d, const int* __restrict__ cursor, long long capacity, int* __restrict__ overflow) {
    const int r = threadIdx.x;
    if (r < d.n) {
        const int n = cursor[r];
        *d.nrec[r] = n;
        if (n > capacity && overflow != nullptr) atomicOr(overflow, 1);
    }
}

struct SparseSources {
    const int* ids[kSparseMaxPeers];
    const float4* sums[kSparseMaxPeers];
    const int* cnts[kSparseMaxPeers];
    const int* nrec[kSparseMaxPeers];
    int n;
};

__global__ void __launch_bounds__(kThreads)
voxel_sparse_merge_kernel(SparseSources s, long long capacity, float* __restrict__ grid0, int* __restrict__ counts0,
                          long long id_begin, long long id_end, int* __restrict__ overflow, bool occupancy) {
    const long long stride = static_cast<long long>(gridDim.x) * kThreads;
    for (int i = 0; i < s.n; ++i) {
        long long n = *s.nrec[i];
        if (n > capacity) {                                       // the source dropped records: this slab is incomplete
            if (overflow != nullptr && blockIdx.x == 0 && threadIdx.x == 0) atomicOr(overflow, 1);
            n = capacity;
        }
        for (long long k = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x; k < n; k += stride) {
            const long long id = s.ids[i][k];
            if (id < id_begin || id >= id_end) continue;          // nothing a well-formed list contains
            if (s.sums[i] != nullptr) red_add_v4(grid0 + id * 4, __ldcs(s.sums[i] + k));
            if (occupancy) counts0[id] = 1;                       // every writer stores the same value
            else atomicAdd(counts0 + id, __ldcs(s.cnts[i] + k));
        }
    }
}

}  // namespace

extern "C" {

int rc_voxel_sparse_send(const float* grid, const int32_t* counts, int32_t n_dest, const int64_t* id_begin_host,
                         const int64_t* id_end_host, int64_t capacity, void* const* dest_ids, void* const* dest_sums,
                         void* const* dest_counts, void* const* dest_nrec, int32_t* cursors, int32_t* overflow, int device,
                         void* stream) {
    if (n_dest < 0 || n_dest > kSparseMaxPeers || capacity < 0 || capacity >= (1ll << 31)) return RC_ERR_BAD_SHAPE;
    if (n_dest == 0) return RC_OK;
    if (id_begin_host == nullptr || id_end_host == nullptr || dest_ids == nullptr || dest_sums == nullptr ||
        dest_counts == nullptr || dest_nrec == nullptr || cursors == nullptr)
        return RC_ERR_NULL_POINTER;
    SparseDests d{};
    d.n = n_dest;
    long long tiles = 0;
    for (int r = 0; r < n_dest; ++r) {
        if (id_begin_host[r] < 0 || id_end_host[r] < id_begin_host[r] || id_end_host[r] >= (1ll << 31)) return RC_ERR_BAD_SHAPE;
        d.begin[r] = id_begin_host[r];
        d.end[r] = id_end_host[r];
        d.tile0[r] = tiles;
        tiles += (d.end[r] - d.begin[r] + kSparseTile - 1) / kSparseTile;
        d.ids[r] = static_cast<int*>(dest_ids[r]);
        d.sums[r] = static_cast<float4*>(dest_sums[r]);
        d.cnts[r] = static_cast<int*>(dest_counts[r]);
        d.nrec[r] = static_cast<int*>(dest_nrec[r]);
        if (d.ids[r] == nullptr || d.cnts[r] == nullptr || d.nrec[r] == nullptr) return RC_ERR_NULL_POINTER;
        if ((grid != nullptr) != (d.sums[r] != nullptr)) return RC_ERR_NULL_POINTER;   // sums travel exactly when there is a grid
        if (!rc::aligned_to(d.ids[r], 4) || !rc::aligned_to(d.sums[r], 16) || !rc::aligned_to(d.cnts[r], 4) || !rc::aligned_to(d.nrec[r], 4))
            return RC_ERR_BAD_ALIGNMENT;
    }
    d.tile0[n_dest] = tiles;
    if (tiles > 0 && counts == nullptr) return RC_ERR_NULL_POINTER;
    if (!rc::aligned_to(grid, 16) || !rc::aligned_to(counts, 16) || !rc::aligned_to(cursors, 4) || !rc::aligned_to(overflow, 4))
        return RC_ERR_BAD_ALIGNMENT;
    rc::DeviceScope scope(device);
    if (scope.status() != RC_OK) return scope.status();
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    RC_CUDA_TRY(cudaMemsetAsync(cursors, 0, static_cast<size_t>(n_dest) * 4, st));
    if (tiles > 0) {
        long long blocks = (tiles + kThreads / 32 - 1) / (kThreads / 32);
        const long long cap = 16ll * rc::sm_count(device);
        if (blocks > cap) blocks = cap;
        voxel_sparse_send_kernel<<<static_cast<unsigned int>(blocks), kThreads, 0, st>>>(
            reinterpret_cast<const float4*>(grid), counts, d, cursors, capacity);
        const int rc_launch = rc::check_launch();
        if (rc_launch != RC_OK) return rc_launch;
    }
    voxel_sparse_publish_kernel<<<1, 32, 0, st>>>(d, cursors, capacity, overflow);
    return rc::check_launch();
}

int rc_voxel_sparse_merge(int32_t n_src, const void* const* src_ids, const void* const* src_sums, const void* const* src_counts,
                          const void* const* src_nrec, int64_t capacity, float* grid, int32_t* counts, int64_t id_begin,
                          int64_t id_end, int32_t* overflow, uint32_t flags, int device, void* stream) {
    if (n_src < 0 || n_src > kSparseMaxPeers || capacity < 0 || id_begin < 0 || id_end < id_begin) return RC_ERR_BAD_SHAPE;
    if (id_end >= (1ll << 31)) return RC_ERR_TOO_LARGE;
    const long long nvox = id_end - id_begin;
    if (nvox > 0 && counts == nullptr) return RC_ERR_NULL_POINTER;
    if (!rc::aligned_to(grid, 16) || !rc::aligned_to(counts, 4)) return RC_ERR_BAD_ALIGNMENT;
    SparseSources s{};
    s.n = n_src;
    if (n_src > 0 && (src_ids == nullptr || src_sums == nullptr || src_counts == nullptr || src_nrec == nullptr)) return RC_ERR_NULL_POINTER;
    if (grid == nullptr) flags |= RC_VOXEL_NO_NORMALIZE;          // count mode: nothing to normalise
    for (int i = 0; i < n_src; ++i) {
        s.ids[i] = static_cast<const int*>(src_ids[i]);
        s.sums[i] = static_cast<const float4*>(src_sums[i]);
        s.cnts[i] = static_cast<const int*>(src_counts[i]);
        s.nrec[i] = static_cast<const int*>(src_nrec[i]);
        if (s.ids[i] == nullptr || s.cnts[i] == nullptr || s.nrec[i] == nullptr) return RC_ERR_NULL_POINTER;
        if ((grid != nullptr) != (s.sums[i] != nullptr)) return RC_ERR_NULL_POINTER;
        if (!rc::aligned_to(s.ids[i], 4) || !rc::aligned_to(s.sums[i], 16) || !rc::aligned_to(s.cnts[i], 4) || !rc::aligned_to(s.nrec[i], 4))
            return RC_ERR_BAD_ALIGNMENT;
    }
    rc::DeviceScope scope(device);
    if (scope.status() != RC_OK) return scope.status();
    if (n_src > 0 && nvox > 0 && capacity > 0) {
        float* grid0 = grid == nullptr ? nullptr
                                       : reinterpret_cast<float*>(reinterpret_cast<uintptr_t>(grid) - static_cast<uintptr_t>(id_begin) * 16u);
        int* counts0 = reinterpret_cast<int*>(reinterpret_cast<uintptr_t>(counts) - static_cast<uintptr_t>(id_begin) * 4u);
        long long blocks = (capacity + kThreads - 1) / kThreads;
        const long long cap = 8ll * rc::sm_count(device);
        if (blocks > cap) blocks = cap;
        voxel_sparse_merge_kernel<<<static_cast<unsigned int>(blocks), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
            s, capacity, grid0, counts0, id_begin, id_end, overflow, (flags & RC_VOXEL_SPARSE_OCCUPANCY) != 0);
        const int rc_launch = rc::check_launch();
        if (rc_launch != RC_OK) return rc_launch;
    }
    if (!(flags & RC_VOXEL_NO_NORMALIZE) && nvox > 0) return rc_voxel_normalize(grid, counts, 0, nvox, 4, device, stream);
    return RC_OK;
}

}  // extern "C"
