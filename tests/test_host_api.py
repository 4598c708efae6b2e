"""Host-side behaviour that needs no GPU: the library loads and exports every declared symbol,
argument validation returns the documented status codes before any CUDA call, and the Python
surface raises instead of falling back to a CPU path."""
import ctypes
import inspect
import os
import re

import pytest
import torch

import robocache
import robogoat_b200
from robogoat_b200 import _lib, api, ops

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    names = set()
    inc = os.path.join(ROOT, "include")
    for f in os.listdir(inc):
        text = open(os.path.join(inc, f)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names |= set(re.findall(r"\b(rc_[a-z0-9_]+)\s*\(", text))
    return names


def test_library_exports_every_declared_symbol(cuda_lib):
    declared = _declared_symbols()
    assert declared, "no declarations found in include/"
    for name in declared:
        assert hasattr(cuda_lib, name), f"{name} declared in include/ but not exported"
    assert set(_lib.EXPORTED_SYMBOLS) <= declared
    assert cuda_lib.rc_abi_version() == 1


def test_status_strings(cuda_lib):
    assert cuda_lib.rc_strerror(0) == b"ok"
    assert b"dtype" in cuda_lib.rc_strerror(3)
    assert cuda_lib.rc_strerror(12345) == b"unknown status"


def test_argument_validation_needs_no_device(cuda_lib):
    L = cuda_lib
    # bad dtype, bad stream count, negative sizes: rejected before any CUDA call
    assert L.rc_resample(None, None, None, None, 1, 1, 1, 1, 7, 0, None) == 3
    assert L.rc_fuse(None, 0, None, None, 1, 1, 0, 0, None) == 2
    assert L.rc_fuse(None, 3, None, None, 1, 1, 0, 0, None) == 1
    assert L.rc_resample(None, None, None, None, -1, 1, 1, 1, 0, 0, None) == 2
    # empty problems succeed without touching the device
    assert L.rc_resample(None, None, None, None, 0, 5, 5, 5, 0, 0, None) == 0
    assert L.rc_resample(None, None, None, None, 4, 5, 0, 5, 1, 0, None) == 0
    # a source with no rows cannot be interpolated
    assert L.rc_resample(None, None, None, None, 1, 0, 1, 1, 0, 0, None) == 2
    assert L.rc_resample(None, None, None, None, 1, 1, 1, 1, 0, 0, None) == 1
    assert L.rc_resample_brackets(None, None, 0, 3, 3, None, None, None, 0, None) == 0
    assert L.rc_resample_brackets(None, None, 1, 0, 3, None, None, None, 0, None) == 2
    gmin = (ctypes.c_float * 3)(0, 0, 0)
    gs = (ctypes.c_int32 * 3)(4, 4, 4)
    buf = ctypes.create_string_buffer(64)
    assert L.rc_voxelize(None, None, buf, None, 0, 0, gmin, 0.1, gs, 9, 0, 0, None) == 5
    assert L.rc_voxelize(None, None, buf, None, 0, 0, gmin, 0.0, gs, 0, 0, 0, None) == 9
    assert L.rc_voxelize(None, None, buf, None, 0, 0, gmin, float("nan"), gs, 0, 0, 0, None) == 9
    assert L.rc_voxelize(None, None, None, None, 0, 0, gmin, 0.1, gs, 0, 0, 0, None) == 1
    assert L.rc_voxelize(None, None, buf, None, -1, 0, gmin, 0.1, gs, 0, 0, 0, None) == 2
    big = (ctypes.c_int32 * 3)(1 << 24, 4, 4)
    assert L.rc_voxelize(None, None, buf, None, 0, 0, gmin, 0.1, big, 0, 0, 0, None) == 7
    assert L.rc_voxel_normalize(None, None, 0, 0, 4, 0, None) == 0
    assert L.rc_voxel_normalize(None, None, 5, 2, 4, 0, None) == 2
    assert L.rc_voxel_normalize(None, None, 0, 8, 4, 0, None) == 1


def test_public_surface_matches_reference_names():
    expected = ["resample_trajectories", "fuse_multimodal", "voxelize_pointcloud", "voxelize_occupancy",
                "is_cuda_available", "check_installation", "self_test", "print_installation_info", "__version__"]
    assert list(robocache.__all__) == expected
    for n in expected:
        assert hasattr(robocache, n) and hasattr(robogoat_b200, n)
    sig = inspect.signature(robocache.resample_trajectories)
    assert list(sig.parameters) == ["source_data", "source_times", "target_times", "device", "backend"]
    sig = inspect.signature(robocache.fuse_multimodal)
    assert list(sig.parameters) == ["stream1_data", "stream1_times", "stream2_data", "stream2_times",
                                    "stream3_data", "stream3_times", "target_times", "backend"]
    sig = inspect.signature(robocache.voxelize_pointcloud)
    assert list(sig.parameters) == ["points", "features", "grid_min", "voxel_size", "grid_size", "mode", "backend"]
    assert sig.parameters["grid_min"].default == [-10.0, -10.0, -10.0]
    assert sig.parameters["voxel_size"].default == 0.1
    assert sig.parameters["grid_size"].default == [128, 128, 128]
    assert sig.parameters["mode"].default == "occupancy"


def test_no_cpu_fallback():
    src, st, tt = torch.zeros(1, 2, 3), torch.zeros(1, 2), torch.zeros(1, 2)
    with pytest.raises(RuntimeError, match="tensors are on CPU"):
        robocache.resample_trajectories(src, st, tt)
    with pytest.raises(RuntimeError, match="pytorch"):
        robocache.resample_trajectories(src, st, tt, backend="pytorch")
    with pytest.raises(ValueError, match="Unknown backend"):
        robocache.resample_trajectories(src, st, tt, backend="invalid")
    with pytest.raises(ValueError, match="Unknown backend"):
        robocache.fuse_multimodal(src, st, src, st, src, st, tt, backend="triton")
    with pytest.raises(RuntimeError, match="tensors are on CPU"):
        robocache.fuse_multimodal(src, st, src, st, src, st, tt)
    with pytest.raises(RuntimeError, match="tensors are on CPU"):
        robocache.voxelize_pointcloud(torch.zeros(4, 3))
    with pytest.raises(RuntimeError, match="must be CUDA tensor"):
        ops.resample_trajectories_cuda(src, st, tt)
    with pytest.raises(RuntimeError, match="must be on CUDA device"):
        ops.voxelize_pointcloud_cuda(torch.zeros(4, 3), None, [0, 0, 0], 0.1, [4, 4, 4], "count")


def test_product_code_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "robogoat_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "import oracle" not in text and "from oracle" not in text, f
    assert "oracle" not in open(os.path.join(ROOT, "robocache", "__init__.py")).read()


def test_check_installation_keys():
    info = robocache.check_installation()
    assert set(info) == {"cuda_extension_available", "multimodal_extension_available", "voxelize_extension_available",
                         "pytorch_available", "cuda_device_available", "gpu_name"}
    assert info["cuda_extension_available"] is True
