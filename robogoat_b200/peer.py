"""Device buffers that the other ranks of a node can write into directly.

``PeerBuffer`` owns one allocation on this rank's GPU and, after ``connect``, holds the device
addresses under which this process can reach every other rank's allocation (CUDA IPC, peer access
over NVLink).  Creation and ``connect`` are collective set-up steps; nothing here runs per step.
Kernels only ever *store* into a peer's buffer; ordering between the writer's kernel and the owner's
reader is the caller's job (a collective on the stream between the two).
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch
import torch.distributed as dist

from . import _lib


class PeerBuffer:
    def __init__(self, nbytes: int, device: Optional[torch.device] = None):
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.nbytes = int(nbytes)
        ptr = ctypes.c_void_p()
        handle = ctypes.create_string_buffer(64)
        _lib.check(_lib.load().rc_peer_alloc(self.nbytes, self.device.index, ctypes.byref(ptr), handle), "peer_alloc")
        self.ptr = int(ptr.value)
        self.handle = bytes(handle.raw)
        self.peers: List[int] = []          # address of every rank's buffer as seen from this process
        self._opened: List[int] = []
        self._group = None
        self._connect_called = False

    def connect(self, group=None) -> None:
        """Collective: exchange the handles and map every other rank's buffer."""
        self._group = group
        self._connect_called = True
        rank, ws = dist.get_rank(group), dist.get_world_size(group)
        handles: List[Optional[bytes]] = [None] * ws
        dist.all_gather_object(handles, self.handle, group=group)
        L = _lib.load()
        self.peers = []
        for r, h in enumerate(handles):
            if r == rank:
                self.peers.append(self.ptr)
                continue
            p = ctypes.c_void_p()
            _lib.check(L.rc_peer_open(h, self.device.index, ctypes.byref(p)), "peer_open")
            self.peers.append(int(p.value))
            self._opened.append(int(p.value))

    def close(self) -> None:
        """Collective when connected: unmap the peers' buffers, wait for everyone, then free the own one."""
        L = _lib.load()
        torch.cuda.synchronize(self.device)
        for p in self._opened:
            L.rc_peer_close(p, self.device.index)
        self._opened = []
        if self._connect_called and dist.is_initialized():   # every rank that connected takes part, mapped or not
            dist.barrier(group=self._group)
        self._connect_called = False
        self.peers = []
        if self.ptr:
            L.rc_peer_free(self.ptr, self.device.index)
            self.ptr = 0
