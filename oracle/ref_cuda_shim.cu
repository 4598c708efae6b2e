// C-ABI shim around the reference's own CUDA launchers, used only as a comparator: a second check
// of the new kernels against the reference's GPU outputs where the two agree by design, and the
// "reference kernels on this GPU" timings of the benchmark's reference arm.  TEST INFRASTRUCTURE ONLY.
//
// The reference sources are compiled from where they lie in the reference checkout
// (robocache/csrc/cuda/{resample,multimodal,voxelize}_kernel.cu, passed to nvcc by the Makefile, with
// the reference's own flags -O3 --use_fast_math but for sm_100a); nothing is copied into this
// repository.  The resample launchers are already extern "C" there
// (robocache/csrc/cuda/resample_kernel.cu:127-174); the other two have C++ linkage and are forwarded.
#include <cuda_runtime.h>

// robocache/csrc/cuda/voxelize_kernel.cu:20-25
enum VoxelMode { COUNT = 0, OCCUPANCY = 1, MEAN = 2, MAX = 3 };

// robocache/csrc/cuda/multimodal_kernel.cu:201-217
void multimodal_fusion_cuda(const void* stream1_data, const float* stream1_times, const void* stream2_data,
                            const float* stream2_times, const void* stream3_data, const float* stream3_times,
                            const float* target_times, void* output, int batch_size, int s1, int d1, int s2, int d2,
                            int s3, int d3, int target_len, bool use_bf16, cudaStream_t stream);

// robocache/csrc/cuda/voxelize_kernel.cu:210-222
void voxelize_cuda(const float* points, const float* features, void* voxel_grid, void* voxel_counts, int num_points,
                   int num_features, float3 grid_min, float voxel_size, int grid_x, int grid_y, int grid_z,
                   VoxelMode mode, cudaStream_t stream);

extern "C" {

void refcuda_fuse(const void* d1, const float* t1, const void* d2, const float* t2, const void* d3, const float* t3,
                  const float* tt, void* out, int B, int s1, int w1, int s2, int w2, int s3, int w3, int T, int use_bf16,
                  void* stream) {
    multimodal_fusion_cuda(d1, t1, d2, t2, d3, t3, tt, out, B, s1, w1, s2, w2, s3, w3, T, use_bf16 != 0,
                           static_cast<cudaStream_t>(stream));
}

void refcuda_voxelize(const float* points, const float* features, void* grid, void* counts, int N, int F, float minx,
                      float miny, float minz, float voxel_size, int gx, int gy, int gz, int mode, void* stream) {
    voxelize_cuda(points, features, grid, counts, N, F, make_float3(minx, miny, minz), voxel_size, gx, gy, gz,
                  static_cast<VoxelMode>(mode), static_cast<cudaStream_t>(stream));
}

}  // extern "C"
