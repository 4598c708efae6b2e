// Status strings, ABI version and the per-device SM-count cache.
#include "rc_common.cuh"

#include <atomic>
#include <map>
#include <mutex>
#include <utility>

namespace rc {

thread_local int g_last_cuda_error = 0;
std::atomic<int> g_allow_block_kernel{1};
std::atomic<int> g_voxel_passes{0};
std::atomic<int> g_part_aligned_store{1};
std::atomic<int> g_bulk_wait_limit{-1};
std::atomic<int> g_gather_bulk_stage{1};
std::atomic<int> g_bucket_bulk_store{1};
std::atomic<int> g_scatter_overlap{1};

// SM count per device, filled on first use (immutable hardware facts, not call state).
static std::atomic<int> g_sm_count[64];

int sm_count(int device) {
    if (device < 0 || device >= 64) return 148;
    int v = g_sm_count[device].load(std::memory_order_relaxed);
    if (v > 0) return v;
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n <= 0) {
        cudaGetLastError();
        n = 148;
    }
    g_sm_count[device].store(n, std::memory_order_relaxed);
    return n;
}

int ensure_dynamic_smem(const void* kernel, int device, size_t bytes) {
    static std::mutex mu;
    static std::map<std::pair<const void*, int>, size_t> granted;
    std::lock_guard<std::mutex> lock(mu);
    size_t& have = granted[std::make_pair(kernel, device)];
    if (have >= bytes) return RC_OK;
    const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes));
    if (e != cudaSuccess) return cuda_fail(e);
    have = bytes;
    return RC_OK;
}

}  // namespace rc

extern "C" {

const char* rc_strerror(int status) {
    switch (status) {
        case RC_OK: return "ok";
        case RC_ERR_NULL_POINTER: return "a required pointer is NULL";
        case RC_ERR_BAD_SHAPE: return "bad shape";
        case RC_ERR_BAD_DTYPE: return "Unsupported dtype. Use float32 or bfloat16.";
        case RC_ERR_BAD_ALIGNMENT: return "pointer is not aligned to its element size";
        case RC_ERR_BAD_MODE: return "invalid voxel mode or missing features";
        case RC_ERR_CUDA: return "CUDA runtime error";
        case RC_ERR_TOO_LARGE: return "size exceeds the supported range";
        case RC_ERR_BAD_DEVICE: return "device index out of range";
        case RC_ERR_BAD_VALUE: return "voxel_size must be positive";
        default: return "unknown status";
    }
}

int rc_last_cuda_error(void) { return rc::g_last_cuda_error; }

int rc_abi_version(void) { return RC_ABI_VERSION; }

int rc_set_option(int option, int value) {
    if (option == RC_OPT_BLOCK_KERNEL) {
        rc::g_allow_block_kernel.store(value != 0, std::memory_order_relaxed);
        return RC_OK;
    }
    if (option == RC_OPT_VOXEL_PASSES) {
        if (value < 0 || value > 64) return RC_ERR_BAD_VALUE;
        rc::g_voxel_passes.store(value, std::memory_order_relaxed);
        return RC_OK;
    }
    if (option == RC_OPT_PART_ALIGNED_STORE) {
        if (value < 0 || value > 2) return RC_ERR_BAD_VALUE;
        rc::g_part_aligned_store.store(value, std::memory_order_relaxed);
        return RC_OK;
    }
    if (option == RC_OPT_GATHER_BULK_STAGE) {
        rc::g_gather_bulk_stage.store(value != 0, std::memory_order_relaxed);
        return RC_OK;
    }
    if (option == RC_OPT_BUCKET_BULK_STORE) {
        rc::g_bucket_bulk_store.store(value != 0, std::memory_order_relaxed);
        return RC_OK;
    }
    if (option == RC_OPT_SCATTER_OVERLAP) {
        rc::g_scatter_overlap.store(value != 0, std::memory_order_relaxed);
        return RC_OK;
    }
    if (option == RC_OPT_BULK_WAIT_LIMIT) {
        if (value < -1) return RC_ERR_BAD_VALUE;
        rc::g_bulk_wait_limit.store(value, std::memory_order_relaxed);
        return RC_OK;
    }
    return RC_ERR_BAD_VALUE;
}

}  // extern "C"
