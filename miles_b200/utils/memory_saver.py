"""Pause / resume device memory by tag without changing addresses.

``MemorySaver.region(tag)`` is a context manager: tensors allocated inside it come from the tagged
virtual-memory arena of the extension (``csrc/vmm_allocator.cpp``: cuMemAddressReserve + cuMemCreate + cuMemMap
behind PyTorch's pluggable-allocator interface). ``pause(tag)`` releases their physical memory (optionally
keeping a host copy), ``resume(tag)`` maps new memory at the same addresses, so tensors, captured CUDA graphs
and kernels holding the pointers stay valid. Paused memory must not be touched until it is resumed.

Reference: torch_memory_saver ``pause/resume(tag)`` used for ``--offload-train`` / ``--offload-rollout``
(miles/backends/megatron_utils/actor.py:299-341; miles/ray/train/actor_factory.py:44-60).
"""
from __future__ import annotations

import contextlib

import torch


class MemorySaver:
    _instance = None

    def __new__(cls):
        if cls._instance is None:
            cls._instance = super().__new__(cls)
            cls._instance._init()
        return cls._instance

    def _init(self) -> None:
        from ..ops import _ext

        self.C = _ext.load(required=True)
        self.available = bool(self.C.vmm_available()) and torch.cuda.is_available()
        self._alloc = None
        self._pools: dict = {}

    def _allocator(self):
        if self._alloc is None:
            self._alloc = torch.cuda.memory.CUDAPluggableAllocator(self.C.__file__, "mb_vmm_malloc", "mb_vmm_free")
        return self._alloc

    @contextlib.contextmanager
    def region(self, tag: str):
        """Allocations made inside the block belong to ``tag``."""
        if not self.available:
            yield
            return
        pool = self._pools.get(tag)
        if pool is None:
            pool = torch.cuda.MemPool(self._allocator().allocator())
            self._pools[tag] = pool
        self.C.vmm_set_tag(tag)
        with torch.cuda.use_mem_pool(pool):
            yield
        self.C.vmm_set_tag("default")

    def pause(self, tag: str, keep_contents: bool = False) -> int:
        """Releases the physical memory of the tag; returns the number of bytes released."""
        return int(self.C.vmm_pause(tag, keep_contents)) if self.available else 0

    def resume(self, tag: str) -> int:
        return int(self.C.vmm_resume(tag)) if self.available else 0

    def stats(self) -> dict:
        return dict(self.C.vmm_stats()) if self.available else {}
