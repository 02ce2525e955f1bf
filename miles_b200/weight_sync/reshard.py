"""Resharding between stores with different expert-parallel layouts (trainer EP -> engine EP)."""
from __future__ import annotations

import torch


def reshard_into(src_store, dst_store, group: str) -> int:
    """Copy parameters by name; expert tensors are sliced by global expert index. Returns bytes moved."""
    moved = 0
    for s in dst_store.specs:
        if s.group != group:
            continue
        dst = dst_store.params[s.name]
        src = src_store.params[s.name]
        if s.group == "expert" and src.shape[0] != dst.shape[0]:
            el_d = dst.shape[0]
            lo = dst_store.ep_rank * el_d - src_store.ep_rank * src.shape[0]
            assert 0 <= lo and lo + el_d <= src.shape[0], "destination experts are not held by this source rank"
            src = src[lo:lo + el_d]
        dst.copy_(src.to(dst.dtype), non_blocking=True)
        moved += dst.numel() * dst.element_size()
    return moved
