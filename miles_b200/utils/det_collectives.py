"""Deterministic reductions for bitwise-reproducibility tests.

``det_all_reduce`` / ``det_reduce_scatter`` replace the backend's reduction order with: all-gather every
rank's contribution, then fold with a fixed pairwise tree (rank order), in chunks so that the gathered
buffer stays bounded.  The result is bitwise identical on every rank and across runs, independent of the
collective algorithm NCCL or gloo would pick.  Reference: miles/utils/test_utils/det_process_group.py:35-317.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

_CHUNK_BYTES = 1 << 30


def _tree_fold(parts: list) -> torch.Tensor:
    while len(parts) > 1:
        nxt = [parts[i] + parts[i + 1] for i in range(0, len(parts) - 1, 2)]
        if len(parts) % 2:
            nxt.append(parts[-1])
        parts = nxt
    return parts[0]


def det_all_reduce(t: torch.Tensor, group: Optional["dist.ProcessGroup"] = None) -> torch.Tensor:
    world = dist.get_world_size(group)
    if world == 1:
        return t
    flat = t.reshape(-1)
    per = max(1, _CHUNK_BYTES // (flat.element_size() * world))
    for a in range(0, flat.numel(), per):
        seg = flat[a:a + per].contiguous()
        bufs = [torch.empty_like(seg) for _ in range(world)]
        dist.all_gather(bufs, seg, group=group)
        flat[a:a + per] = _tree_fold(bufs)
    return t


def det_reduce_scatter(out: torch.Tensor, inp: torch.Tensor, group: Optional["dist.ProcessGroup"] = None) -> torch.Tensor:
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    full = det_all_reduce(inp.clone(), group)
    n = out.numel()
    out.copy_(full.reshape(-1)[rank * n:(rank + 1) * n].view_as(out))
    return out
