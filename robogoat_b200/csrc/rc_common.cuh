// Shared host-side helpers of the C-ABI entry points: status bookkeeping, a scoped device
// switch, pointer-alignment tests and the launch-error check.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "robocache_b200.h"

namespace rc {

// cudaError_t behind the last RC_ERR_CUDA returned on this thread
extern thread_local int g_last_cuda_error;

inline int cuda_fail(cudaError_t e) {
    g_last_cuda_error = static_cast<int>(e);
    return RC_ERR_CUDA;
}

#define RC_CUDA_TRY(expr)                                   \
    do {                                                    \
        cudaError_t rc_e_ = (expr);                         \
        if (rc_e_ != cudaSuccess) return rc::cuda_fail(rc_e_); \
    } while (0)

// Makes `device` current for the scope and restores the caller's device afterwards (the
// reference bindings take no device guard at all: robocache/csrc/cpp/resample_ops.cpp:31-90).
class DeviceScope {
public:
    explicit DeviceScope(int device) : status_(RC_OK), prev_(-1), switched_(false) {
        int count = 0;
        cudaError_t e = cudaGetDeviceCount(&count);
        if (e != cudaSuccess) { status_ = cuda_fail(e); return; }
        if (device < 0 || device >= count) { status_ = RC_ERR_BAD_DEVICE; return; }
        e = cudaGetDevice(&prev_);
        if (e != cudaSuccess) { status_ = cuda_fail(e); return; }
        if (prev_ != device) {
            e = cudaSetDevice(device);
            if (e != cudaSuccess) { status_ = cuda_fail(e); return; }
            switched_ = true;
        }
    }
    ~DeviceScope() {
        if (switched_) cudaSetDevice(prev_);
    }
    int status() const { return status_; }

private:
    int status_;
    int prev_;
    bool switched_;
};

inline bool aligned_to(const void* p, uintptr_t a) {
    return (reinterpret_cast<uintptr_t>(p) % a) == 0;
}

// Launch errors are read without synchronising: cudaPeekAtLastError leaves sticky state
// alone, so a fault raised by unrelated earlier work is still reported to its owner.
inline int check_launch() {
    cudaError_t e = cudaPeekAtLastError();
    if (e != cudaSuccess) {
        cudaGetLastError();  // clear the non-sticky launch error so later calls start clean
        return cuda_fail(e);
    }
    return RC_OK;
}

int sm_count(int device);

// Raises a kernel's dynamic shared-memory limit to `bytes` on `device` (current) once; later calls with
// the same or a smaller size return without touching the runtime, so launches stay capturable.
int ensure_dynamic_smem(const void* kernel, int device, size_t bytes);

// process-wide switches behind rc_set_option
extern std::atomic<int> g_allow_block_kernel;  // RC_OPT_BLOCK_KERNEL
extern std::atomic<int> g_voxel_passes;        // RC_OPT_VOXEL_PASSES
extern std::atomic<int> g_part_aligned_store;     // RC_OPT_PART_ALIGNED_STORE
extern std::atomic<int> g_gather_bulk_stage;      // RC_OPT_GATHER_BULK_STAGE
extern std::atomic<int> g_bucket_bulk_store;      // RC_OPT_BUCKET_BULK_STORE
extern std::atomic<int> g_scatter_overlap;        // RC_OPT_SCATTER_OVERLAP
extern std::atomic<int> g_bulk_wait_limit;        // RC_OPT_BULK_WAIT_LIMIT (-1 = built-in limit)

}  // namespace rc
