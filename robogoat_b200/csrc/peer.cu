// Device buffers that other processes of the same node can map (CUDA IPC), for the kernels that
// write straight into a peer GPU's memory.  Allocation and mapping are explicit calls made once,
// outside any hot path; nothing here runs per step - except the barrier at the end of this file, which
// is one tiny kernel per call.
#include <cstring>

#include "rc_common.cuh"

namespace {

constexpr int kBarrierMaxRanks = 16;
constexpr long long kBarrierDefaultPolls = 1ll << 25;      // about 8 s of polling (0.26 us per poll): ranks may be seconds apart

struct BarrierFlags {
    unsigned int* arr[kBarrierMaxRanks];    // arr[p]: rank p's flag array (uint32 [n]) as mapped into this process
    int n, rank;
};

// One thread per rank p: tell p that this rank has arrived (a release store of the epoch into slot `rank` of p's
// array, after a system-scope fence so that everything this GPU wrote before - including plain stores into peers'
// memory by earlier kernels of the stream - is performed first), then wait until p's arrival shows up in this rank's
// own array.  The wait is bounded: after poll_limit polls the thread raises *status and gives up, so a rank that
// never arrives costs the others a few seconds and an error code, not a hung GPU.  Epochs only grow (compared as a
// signed difference, so they may wrap); a fast rank's next epoch satisfies a slow rank's wait for this one.
__global__ void peer_barrier_kernel(BarrierFlags f, unsigned int epoch, long long poll_limit, int* status) {
    const int p = threadIdx.x;
    if (p < f.n) {
        __threadfence_system();
        asm volatile("st.release.sys.global.u32 [%0], %1;" :: "l"(f.arr[p] + f.rank), "r"(epoch) : "memory");
        const unsigned int* mine = f.arr[f.rank] + p;
        for (long long it = 0;; ++it) {
            unsigned int v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
            if (static_cast<int>(v - epoch) >= 0) break;
            if (it >= poll_limit) {
                if (status != nullptr) atomicExch(status, 1);
                break;
            }
            __nanosleep(100);
        }
    }
    __syncthreads();
    __threadfence_system();
}

}  // namespace

extern "C" {

int rc_peer_barrier(void* const* flags, int32_t n, int32_t rank, uint32_t epoch, int32_t* status, int64_t poll_limit,
                    int device, void* stream) {
    if (flags == nullptr) return RC_ERR_NULL_POINTER;
    if (n < 1 || n > kBarrierMaxRanks || rank < 0 || rank >= n || poll_limit < 0) return RC_ERR_BAD_SHAPE;
    BarrierFlags f{};
    f.n = n;
    f.rank = rank;
    for (int p = 0; p < n; ++p) {
        f.arr[p] = static_cast<unsigned int*>(flags[p]);
        if (f.arr[p] == nullptr) return RC_ERR_NULL_POINTER;
        if (!rc::aligned_to(f.arr[p], 4)) return RC_ERR_BAD_ALIGNMENT;
    }
    if (!rc::aligned_to(status, 4)) return RC_ERR_BAD_ALIGNMENT;
    rc::DeviceScope scope(device);
    if (scope.status() != RC_OK) return scope.status();
    peer_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(f, epoch, poll_limit > 0 ? poll_limit : kBarrierDefaultPolls,
                                                                         status);
    return rc::check_launch();
}

int rc_peer_alloc(uint64_t bytes, int device, void** ptr, unsigned char handle[64]) {
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    if (ptr == nullptr || handle == nullptr) return RC_ERR_NULL_POINTER;
    if (bytes == 0) return RC_ERR_BAD_SHAPE;
    rc::DeviceScope scope(device);
    if (scope.status() != RC_OK) return scope.status();
    void* p = nullptr;
    RC_CUDA_TRY(cudaMalloc(&p, bytes));
    cudaError_t e = cudaMemset(p, 0, bytes);            // flag arrays of rc_peer_barrier must start at zero
    if (e != cudaSuccess) {
        cudaFree(p);
        return rc::cuda_fail(e);
    }
    cudaIpcMemHandle_t h;
    e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
        cudaFree(p);
        return rc::cuda_fail(e);
    }
    std::memcpy(handle, &h, 64);
    *ptr = p;
    return RC_OK;
}

int rc_peer_open(const unsigned char handle[64], int device, void** ptr) {
    if (ptr == nullptr || handle == nullptr) return RC_ERR_NULL_POINTER;
    rc::DeviceScope scope(device);
    if (scope.status() != RC_OK) return scope.status();
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle, 64);
    void* p = nullptr;
    RC_CUDA_TRY(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    *ptr = p;
    return RC_OK;
}

int rc_peer_close(void* ptr, int device) {
    if (ptr == nullptr) return RC_OK;
    rc::DeviceScope scope(device);
    if (scope.status() != RC_OK) return scope.status();
    RC_CUDA_TRY(cudaIpcCloseMemHandle(ptr));
    return RC_OK;
}

int rc_peer_free(void* ptr, int device) {
    if (ptr == nullptr) return RC_OK;
    rc::DeviceScope scope(device);
    if (scope.status() != RC_OK) return scope.status();
    RC_CUDA_TRY(cudaFree(ptr));
    return RC_OK;
}

}  // extern "C"
