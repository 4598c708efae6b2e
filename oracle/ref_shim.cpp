// C-ABI shim around the reference's own C++ CPU header, used only to validate the
// oracle.  TEST INFRASTRUCTURE ONLY.
//
// The header is compiled from where it lies in the reference checkout
// (robocache/validation/cpu_reference.hpp, found through the -I path the Makefile
// passes); no reference source is copied into this repository.  The built library goes
// to oracle/_ref/ and is never loaded by the shipped package.
#include "cpu_reference.hpp"

extern "C" {

// robocache/validation/cpu_reference.hpp:180-216 — batched float occupancy, z-major
void ref_voxelize_occupancy(const float* points, float* grid, int batch, int num_points,
                            int depth, int height, int width, float voxel_size,
                            const float* origin) {
    robocache::validation::cpu_voxelize_occupancy(points, grid, batch, num_points, depth, height,
                                                  width, voxel_size, origin);
}

// robocache/validation/cpu_reference.hpp:221-250 — batched float point counts
void ref_voxelize_density(const float* points, float* grid, int batch, int num_points,
                          int depth, int height, int width, float voxel_size,
                          const float* origin) {
    robocache::validation::cpu_voxelize_density(points, grid, batch, num_points, depth, height,
                                                width, voxel_size, origin);
}

// robocache/validation/cpu_reference.hpp:30-75 — the header's resample variant.  It uses
// a different bracket rule and lerp form from the torch path the oracle follows, so it
// is exported only to document that divergence in a test, not as a parity target.
void ref_resample_f32(const float* src, const float* st, const float* tt, float* out,
                      int B, int S, int T, int D) {
    robocache::validation::cpu_resample_trajectories<float>(src, st, tt, out, B, S, T, D);
}

}  // extern "C"
