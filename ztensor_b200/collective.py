"""Peer-mapped buffers of the all-reduce that is fused into row-parallel GEMVs.

One process per GPU.  Every rank allocates its slot buffer and state words with the library's own allocator, exports CUDA IPC handles, and the
handles are exchanged over the process group (host side, gloo or nccl object
collectives).  The result is the ZtqAllReduce descriptor of include/ztq.h.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from . import _lib


class ZtqAllReduce(C.Structure):
    _fields_ = [("world", C.c_int), ("rank", C.c_int), ("slot_stride", C.c_int), ("reserved", C.c_int),
                ("slots", C.c_void_p * 8), ("state", C.c_void_p)]


def _alloc(nbytes: int) -> int:
    p = C.c_void_p()
    _lib.check(_lib.lib().ztq_symm_alloc(C.byref(p), nbytes), "ztq_symm_alloc")
    return p.value


def _export(ptr: int) -> bytes:
    buf = C.create_string_buffer(64)
    _lib.check(_lib.lib().ztq_ipc_export(ptr, buf), "ztq_ipc_export")
    return buf.raw


def _open(handle: bytes) -> int:
    p = C.c_void_p()
    _lib.check(_lib.lib().ztq_ipc_open(C.create_string_buffer(handle, 64), C.byref(p)), "ztq_ipc_open")
    return p.value


class FusedAllReduce:
    """Owns the symmetric buffers of one rank and the mappings of its peers."""

    def __init__(self, max_elems: int, group=None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if not 2 <= self.world <= 8:
            raise ValueError("fused all-reduce supports 2..8 ranks of one node")
        self.slot_stride = (max_elems + 31) // 32 * 32
        self._sizes = [2 * self.world * self.slot_stride * 8, 16]
        self._own = [_alloc(n) for n in self._sizes]
        handles = [None] * self.world
        dist.all_gather_object(handles, _export(self._own[0]), group=group)
        self._peer = []
        self.desc = ZtqAllReduce()
        self.desc.world, self.desc.rank = self.world, self.rank
        self.desc.slot_stride = self.slot_stride
        for r, hs in enumerate(handles):
            if r == self.rank:
                self.desc.slots[r] = self._own[0]
            else:
                ps = _open(hs)
                self._peer.append(ps)
                self.desc.slots[r] = ps
        self.desc.state = self._own[1]
        dist.barrier(group=group)          # every rank has mapped every buffer before the first push

    def ptr(self):
        return C.byref(self.desc)

    def resync(self):
        """Bring all ranks back to launch sequence 0.  Needed after a launch that gave up on a peer (device error
        4): the ranks' sequence numbers may then disagree for good.  Every rank calls this between steps, with no
        kernel of its own in flight: meet, zero the own slot buffer and state words, meet again."""
        torch.cuda.synchronize()
        dist.barrier(group=self.group)     # nobody pushes any more
        for p, n in zip(self._own, self._sizes):
            _lib.check(_lib.lib().ztq_symm_zero(p, n), "ztq_symm_zero")
        dist.barrier(group=self.group)     # every buffer is clean before the next push

    def close(self):
        torch.cuda.synchronize()
        dist.barrier(group=self.group)     # nobody is still pushing into a buffer that is about to go
        for p in self._peer:
            _lib.lib().ztq_ipc_close(p)
        for p in self._own:
            _lib.lib().ztq_symm_free(p)
        self._peer, self._own = [], []
