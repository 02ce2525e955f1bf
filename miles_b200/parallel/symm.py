"""Symmetric device memory: one allocation per rank that every peer of a process group maps.

The region is allocated with plain ``cudaMalloc`` by the extension, exported as a CUDA IPC handle,
exchanged over the group and opened by each peer, which yields one device pointer per rank for the same
logical buffer.  Kernels then read / write peer memory with ordinary loads and stores over NVLink (no
TMA multicast, no library collectives).  Sub-buffers are carved out at identical offsets on all ranks.
"""
from __future__ import annotations


import torch
import torch.distributed as dist

from ..ops import _ext


class SymmetricRegion:
    def __init__(self, nbytes: int, group, rank: int, world: int, device: torch.device):
        self.C = _ext.load(required=True)
        self.nbytes = int((nbytes + 255) // 256 * 256)
        self.group, self.rank, self.world, self.device = group, rank, world, device
        self.base, handle = self.C.symm_alloc(self.nbytes)
        handles = [None] * world
        dist.all_gather_object(handles, bytes(handle), group=group)
        self.peer_base = []
        for r in range(world):
            self.peer_base.append(self.base if r == rank else self.C.symm_open(handles[r]))
        self._cursor = 0
        dist.barrier(group=group)

    def carve(self, shape, dtype: torch.dtype, align: int = 256):
        """Returns (local tensor view, [peer addresses]) of a sub-buffer at the same offset on every rank."""
        n = 1
        for s in shape:
            n *= int(s)
        nb = n * torch.empty((), dtype=dtype).element_size()
        off = (self._cursor + align - 1) // align * align
        assert off + nb <= self.nbytes, "symmetric region exhausted"
        self._cursor = off + nb
        t = self.C.tensor_from_ptr(self.base + off, list(shape), dtype, self.device.index or 0)
        return t, [b + off for b in self.peer_base]

    def close(self) -> None:
        for r, b in enumerate(self.peer_base):
            if r != self.rank:
                self.C.symm_close(b)
        self.C.symm_free(self.base)
        self.peer_base = []
