// Device buffers that other processes of the same node can map (CUDA IPC), for the kernels that
// write straight into a peer GPU's memory.  Allocation and mapping are explicit calls made once,
// outside any hot path; nothing here runs per step.
#include <cstring>

#include "rc_common.cuh"

extern "C" {

int rc_peer_alloc(uint64_t bytes, int device, void** ptr, unsigned char handle[64]) {
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    if (ptr == nullptr || handle == nullptr) return RC_ERR_NULL_POINTER;
    if (bytes == 0) return RC_ERR_BAD_SHAPE;
    rc::DeviceScope scope(device);
    if (scope.status() != RC_OK) return scope.status();
    void* p = nullptr;
    RC_CUDA_TRY(cudaMalloc(&p, bytes));
    cudaIpcMemHandle_t h;
    const cudaError_t e = cudaIpcGetMemHandle(&h, p);
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
