"""Host-buffer entry points: inputs and outputs live in (pinned) host memory.

``resample_trajectories_host`` is what a caller with CPU-side trajectories uses: it cuts the batch into
row chunks and keeps three CUDA streams busy — host→device copies of chunk c+1, the resample kernel on
chunk c and the device→host copy of chunk c-1 run concurrently — so a call costs about
max(H2D, D2H, kernel) instead of their sum.  Batch rows are independent, so chunking changes no bits.

Device staging buffers are torch tensors cached per (device, shape, dtype) between calls; streams and
events are torch's.  The kernels are the same C-ABI calls the device-tensor API makes.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from . import _lib

_NBUF = 3  # chunks in flight: one being uploaded, one computed, one downloaded


class _Stage:
    """Per-device streams, events and staging buffers of the pipeline."""

    def __init__(self, device: torch.device):
        self.device = device
        self.h2d = torch.cuda.Stream(device)
        self.compute = torch.cuda.Stream(device)
        self.d2h = torch.cuda.Stream(device)
        self.buffers: Dict[Tuple, list] = {}

    def get(self, rows: int, S: int, T: int, D: int, dtype: torch.dtype):
        key = (rows, S, T, D, dtype)
        if key not in self.buffers:
            self.buffers.clear()  # one working shape at a time keeps the footprint bounded
            dev = self.device
            self.buffers[key] = [dict(
                src=torch.empty((rows, S, D), dtype=dtype, device=dev),
                st=torch.empty((rows, S), dtype=torch.float32, device=dev),
                tt=torch.empty((rows, T), dtype=torch.float32, device=dev),
                out=torch.empty((rows, T, D), dtype=dtype, device=dev),
                uploaded=torch.cuda.Event(), computed=torch.cuda.Event(), downloaded=torch.cuda.Event(),
            ) for _ in range(_NBUF)]
        return self.buffers[key]


_stages: Dict[int, _Stage] = {}


def _stage(device: torch.device) -> _Stage:
    if device.index not in _stages:
        _stages[device.index] = _Stage(device)
    return _stages[device.index]


def _host_f32(t: torch.Tensor) -> torch.Tensor:
    return t if (t.dtype == torch.float32 and t.is_contiguous()) else t.to(torch.float32).contiguous()


def resample_trajectories_host(source_data: torch.Tensor, source_times: torch.Tensor, target_times: torch.Tensor,
                               out: Optional[torch.Tensor] = None, device=None, chunk_rows: int = 256) -> torch.Tensor:
    """Resample CPU-resident trajectories on the GPU; returns a pinned CPU tensor [B, T, D].

    Same semantics as ``resample_trajectories``.  Inputs should be pinned for full copy speed (pageable
    memory works, slower).  ``out`` may be a preallocated pinned tensor.  The call returns after the last
    chunk has landed in ``out``.
    """
    if source_data.is_cuda or source_times.is_cuda or target_times.is_cuda:
        raise RuntimeError("resample_trajectories_host takes CPU tensors; use resample_trajectories for CUDA tensors")
    if source_data.dim() != 3 or source_times.dim() != 2 or target_times.dim() != 2:
        raise RuntimeError("source_data must be 3D [B, S, D]; times must be 2D")
    B, S, D = source_data.shape
    T = target_times.shape[1]
    if source_times.shape != (B, S) or target_times.shape[0] != B:
        raise RuntimeError("Batch size mismatch" if source_times.shape[0] != B or target_times.shape[0] != B
                           else "Source length mismatch")
    if source_data.dtype == torch.bfloat16:
        code = _lib.RC_DTYPE_BF16
    elif source_data.dtype == torch.float32:
        code = _lib.RC_DTYPE_F32
    else:
        raise RuntimeError("Unsupported dtype. Use float32 or bfloat16.")
    L = _lib.load()
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    if dev.index is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    src = source_data.contiguous()
    st, tt = _host_f32(source_times), _host_f32(target_times)
    if out is None:
        out = torch.empty((B, T, D), dtype=source_data.dtype).pin_memory()
    elif out.shape != (B, T, D) or out.dtype != source_data.dtype or not out.is_contiguous() or out.is_cuda:
        raise RuntimeError("out must be a contiguous CPU tensor [B, T, D] of the input dtype")
    if B == 0 or T == 0 or D == 0:
        return out
    if S == 0:
        raise RuntimeError("source_data must have at least one timestep")

    rows = max(1, min(int(chunk_rows), B))
    stage = _stage(dev)
    bufs = stage.get(rows, S, T, D, source_data.dtype)
    n_chunks = (B + rows - 1) // rows
    for c in range(n_chunks):
        a, b = c * rows, min(B, (c + 1) * rows)
        n = b - a
        buf = bufs[c % _NBUF]
        with torch.cuda.stream(stage.h2d):
            if c >= _NBUF:
                stage.h2d.wait_event(buf["computed"])       # the kernel that read this buffer's inputs is done
            buf["src"][:n].copy_(src[a:b], non_blocking=True)
            buf["st"][:n].copy_(st[a:b], non_blocking=True)
            buf["tt"][:n].copy_(tt[a:b], non_blocking=True)
            buf["uploaded"].record(stage.h2d)
        with torch.cuda.stream(stage.compute):
            stage.compute.wait_event(buf["uploaded"])
            if c >= _NBUF:
                stage.compute.wait_event(buf["downloaded"])  # the previous result in this buffer has left
            rc = L.rc_resample(buf["src"].data_ptr(), buf["st"].data_ptr(), buf["tt"].data_ptr(), buf["out"].data_ptr(),
                               n, S, T, D, code, dev.index, stage.compute.cuda_stream)
            _lib.check(rc, "resample_trajectories_host")
            buf["computed"].record(stage.compute)
        with torch.cuda.stream(stage.d2h):
            stage.d2h.wait_event(buf["computed"])
            out[a:b].copy_(buf["out"][:n], non_blocking=True)
            buf["downloaded"].record(stage.d2h)
    stage.d2h.synchronize()
    return out
