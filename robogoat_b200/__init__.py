"""B200-native (sm_100a) implementation of RoboCache's preprocessing hot path.

Timestamp-aligned trajectory resampling, multimodal temporal fusion and point-cloud
voxelisation behind the reference's Python operator API.  The CUDA kernels live in
``csrc/`` and are reached through a C-ABI shared library (``include/robocache_b200.h``).
"""
from .api import (  # noqa: F401
    __version__,
    check_installation,
    fuse_multimodal,
    is_cuda_available,
    print_installation_info,
    resample_trajectories,
    self_test,
    voxelize_occupancy,
    voxelize_pointcloud,
)

from .host_pipeline import resample_trajectories_host  # noqa: E402,F401  (host-buffer entry point, not part of the reference API)

__all__ = [
    "resample_trajectories", "fuse_multimodal", "voxelize_pointcloud", "voxelize_occupancy",
    "is_cuda_available", "check_installation", "self_test", "print_installation_info", "__version__",
]
