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


class PeerBarrier:
    """Barrier among the ranks of a node on the current CUDA stream, without NCCL: one 32-thread kernel per call that
    stores an epoch into every peer's flag array over NVLink and polls its own (``rc_peer_barrier``).  Work enqueued
    after ``wait()`` on any rank sees what every rank's stream did before its ``wait()``, plain stores into peers'
    memory included.  The kernel's wait is bounded (about 8 seconds by default): a rank that never arrives raises
    ``status`` on the others instead of hanging them - read it with ``timed_out()``.  Construction and ``close`` are
    collective; every rank must call ``wait()`` the same number of times."""

    def __init__(self, group=None, device: Optional[torch.device] = None, poll_limit: int = 0):
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if self.world > 16:
            raise RuntimeError("the peer barrier supports at most 16 ranks")
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.poll_limit = int(poll_limit)
        self.epoch = 0
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.flags = PeerBuffer(128, self.device)       # zero-filled by the allocation
        self.flags.connect(group)
        dist.barrier(group=group)                       # nobody signals before everybody has mapped

    def wait(self) -> None:
        self.epoch += 1
        VP = ctypes.c_void_p * self.world
        rc = _lib.load().rc_peer_barrier(VP(*self.flags.peers), self.world, self.rank, self.epoch & 0xFFFFFFFF,
                                         self.status.data_ptr(), self.poll_limit, self.device.index,
                                         torch.cuda.current_stream(self.device).cuda_stream)
        _lib.check(rc, "peer_barrier")

    def timed_out(self) -> bool:
        """True if any ``wait()`` so far gave up (synchronises with the device)."""
        return bool(int(self.status.item()))

    def close(self) -> None:
        if self.flags is not None:
            self.flags.close()
            self.flags = None
