"""The reference's Python operator surface, kept verbatim, on top of the sm_100a kernels.

Signatures, argument names, shapes, dtypes and output layout follow
robocache/python/robocache/__init__.py:41-281 and :465-480.  Departures, all deliberate:

* there is no CPU / PyTorch fallback: ``backend='pytorch'`` and CPU tensors raise
  ``RuntimeError`` instead of silently switching implementation;
* an unknown ``backend`` raises ``ValueError`` in all three operators (the reference's
  resampler ignores it, its other two operators raise);
* values follow the reference's torch path (clamped weights, ``f_l*(1-w) + f_r*w``), which
  its own CUDA kernels do not do outside the source range.
"""
from __future__ import annotations

import platform
import sys
from typing import Optional, TextIO

import torch

from . import _lib, ops

__version__ = "1.0.0"

_NO_FALLBACK = ("the B200 build has no PyTorch/CPU backend: tensors must be CUDA tensors and backend must be "
                "None or 'cuda'")


def _resolve_backend(backend: Optional[str]) -> None:
    if backend is None or backend == "cuda":
        return
    if backend == "pytorch":
        raise RuntimeError(f"backend='pytorch' requested but {_NO_FALLBACK}")
    raise ValueError(f"Unknown backend: {backend}. Expected 'cuda' or None")


def _require_cuda(t: torch.Tensor) -> None:
    if not _lib.is_built():
        raise RuntimeError("CUDA backend requested but RoboCache CUDA kernels not available. "
                           "Ensure CUDA extension was compiled successfully.")
    if not t.is_cuda:
        raise RuntimeError(f"CUDA backend requested but tensors are on CPU ({_NO_FALLBACK})")


def resample_trajectories(source_data: torch.Tensor, source_times: torch.Tensor, target_times: torch.Tensor,
                          device: Optional[str] = None, backend: Optional[str] = None) -> torch.Tensor:
    """Resample trajectory data from source to target timestamps.

    Args:
        source_data: Input trajectory [B, S, D] (BF16 or FP32)
        source_times: Source timestamps [B, S], sorted ascending per row
        target_times: Target timestamps [B, T] (any order)
        device: Target device (default: source_data.device)
        backend: None or 'cuda'

    Returns:
        Resampled trajectory [B, T, D], dtype of ``source_data``.  Targets outside the source
        range take the first / last row.
    """
    _resolve_backend(backend)
    if device is not None:
        source_data = source_data.to(device)
        source_times = source_times.to(device)
        target_times = target_times.to(device)
    elif source_times.device != source_data.device or target_times.device != source_data.device:
        source_times = source_times.to(source_data.device)   # default: everything follows source_data
        target_times = target_times.to(source_data.device)
    _require_cuda(source_data)
    return ops.resample_trajectories_cuda(source_data, source_times, target_times)


def fuse_multimodal(stream1_data: torch.Tensor, stream1_times: torch.Tensor, stream2_data: torch.Tensor,
                    stream2_times: torch.Tensor, stream3_data: torch.Tensor, stream3_times: torch.Tensor,
                    target_times: torch.Tensor, backend: Optional[str] = None) -> torch.Tensor:
    """Fuse three timestamped sensor streams onto common target timestamps.

    Args:
        streamK_data: [B, SK, DK], all of one dtype (BF16 or FP32)
        streamK_times: [B, SK], sorted ascending per row
        target_times: [B, T]
        backend: None or 'cuda'

    Returns:
        Fused features [B, T, D1+D2+D3]; columns [0,D1) stream 1, [D1,D1+D2) stream 2, rest stream 3.
    """
    _resolve_backend(backend)
    _require_cuda(stream1_data)
    return ops.fuse_multimodal_cuda(stream1_data, stream1_times, stream2_data, stream2_times, stream3_data,
                                    stream3_times, target_times)


def voxelize_pointcloud(points: torch.Tensor, features: Optional[torch.Tensor] = None,
                        grid_min: list = [-10.0, -10.0, -10.0], voxel_size: float = 0.1,
                        grid_size: list = [128, 128, 128], mode: str = "occupancy",
                        backend: Optional[str] = None) -> torch.Tensor:
    """Voxelize a 3D point cloud onto a regular grid.

    Args:
        points: Point coordinates [N, 3] (x, y, z)
        features: Point features [N, F] (required for mean/max modes)
        grid_min: Minimum corner [x, y, z]
        voxel_size: Voxel edge length
        grid_size: Grid dimensions [X, Y, Z]
        mode: "count", "occupancy", "mean", "max"
        backend: None or 'cuda'

    Returns:
        int32 [X, Y, Z] for count/occupancy, float32 [X, Y, Z, F] for mean/max.  Points outside the
        grid are dropped.  As in the reference's CUDA kernels the flat index of voxel (vx,vy,vz) in
        the returned contiguous tensor is vz*X*Y + vy*X + vx.
    """
    _resolve_backend(backend)
    _require_cuda(points)
    results = ops.voxelize_pointcloud_cuda(points, features, list(grid_min), float(voxel_size), list(grid_size), mode)
    return results[0]


def voxelize_occupancy(points, grid_size, voxel_size, origin, backend=None):
    """Compatibility wrapper: ``voxelize_pointcloud(..., mode='occupancy')``."""
    return voxelize_pointcloud(
        points=points, features=None,
        grid_min=origin.tolist() if hasattr(origin, "tolist") else origin,
        voxel_size=voxel_size,
        grid_size=grid_size.tolist() if hasattr(grid_size, "tolist") else grid_size,
        mode="occupancy", backend=backend)


def is_cuda_available() -> bool:
    """True when the CUDA library is built and a CUDA device is present."""
    return _lib.is_built() and torch.cuda.is_available()


def check_installation() -> dict:
    built = _lib.is_built()
    has_gpu = torch.cuda.is_available()
    return {
        "cuda_extension_available": built,
        "multimodal_extension_available": built,
        "voxelize_extension_available": built,
        "pytorch_available": True,
        "cuda_device_available": has_gpu,
        "gpu_name": torch.cuda.get_device_name(0) if has_gpu else None,
    }


def print_installation_info(stream: Optional[TextIO] = None) -> None:
    if stream is None:
        stream = sys.stdout
    info = check_installation()
    lines = [
        "RoboCache Installation Info (B200 build)", "=" * 60, f"Version: {__version__}",
        f"Python: {platform.python_version()}", f"PyTorch: {torch.__version__}",
        f"CUDA available: {info['cuda_device_available']}", f"CUDA runtime: {torch.version.cuda}",
        f"GPU: {info['gpu_name'] or 'N/A'}", f"CUDA kernels loaded: {info['cuda_extension_available']}",
        f"Multimodal kernels loaded: {info['multimodal_extension_available']}",
        f"Voxelize kernels loaded: {info['voxelize_extension_available']}", "Library: " + _lib.LIB_PATH,
    ]
    for line in lines:
        stream.write(line + "\n")


def self_test() -> bool:
    """Functional check of the three operators on cuda:0 against known answers."""
    if not is_cuda_available():
        raise RuntimeError("self_test needs the CUDA library and a CUDA device; there is no CPU mode")
    dev = "cuda"
    for dtype in (torch.float32, torch.bfloat16):
        src = torch.randn(2, 10, 8, dtype=dtype, device=dev)
        st = torch.linspace(0, 1, 10, device=dev).expand(2, -1)
        tt = torch.linspace(0, 1, 5, device=dev).expand(2, -1)
        out = resample_trajectories(src, st, tt)
        assert out.shape == (2, 5, 8) and out.dtype == dtype and not torch.isnan(out.float()).any()
    out = resample_trajectories(torch.tensor([[[1.0], [2.0], [3.0]]], device=dev),
                                torch.tensor([[0.0, 0.5, 1.0]], device=dev), torch.tensor([[0.25, 0.75]], device=dev))
    assert torch.allclose(out, torch.tensor([[[1.5], [2.5]]], device=dev), atol=1e-4)
    pts = torch.rand(1000, 3, device=dev) * 10.0 - 5.0
    grid = voxelize_pointcloud(pts, grid_min=[-5.0, -5.0, -5.0], voxel_size=0.1, grid_size=[100, 100, 100],
                               mode="occupancy")
    assert grid.shape == (100, 100, 100) and grid.sum() > 0
    streams = []
    for n, d in ((10, 64), (20, 32), (40, 12)):
        streams += [torch.randn(2, n, d, device=dev), torch.linspace(0, 1, n, device=dev).expand(2, -1)]
    fused = fuse_multimodal(*streams, torch.linspace(0, 1, 15, device=dev).expand(2, -1))
    assert fused.shape == (2, 15, 108) and not torch.isnan(fused).any()
    try:
        resample_trajectories(src, st, tt, backend="invalid")
        raise AssertionError("invalid backend accepted")
    except (ValueError, RuntimeError):
        pass
    return True


__all__ = [
    "resample_trajectories", "fuse_multimodal", "voxelize_pointcloud", "voxelize_occupancy",
    "is_cuda_available", "check_installation", "self_test", "print_installation_info", "__version__",
]
