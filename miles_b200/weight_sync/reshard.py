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


def gather_experts_into(src_store, dst_store, ep_group) -> int:
    """Trainer holds ``E / ep`` experts per rank, the rollout replica all ``E``: every expert tensor of the replica
    is the all-gather of the ranks' shares along the expert dimension (contiguous chunks, no staging copy).
    Returns the bytes received by this rank."""
    import torch.distributed as dist

    moved = 0
    for s in dst_store.specs:
        if s.group != "expert":
            continue
        dst, src = dst_store.params[s.name], src_store.params[s.name]
        dist.all_gather_into_tensor(dst, src.contiguous(), group=ep_group)
        moved += (dst.numel() - src.numel()) * dst.element_size()
    return moved


def gather_stages_into(src_store, dst_store, pp) -> int:
    """Trainer holds the layers of one pipeline stage, the rollout replica the whole model: every tensor of the
    replica is broadcast inside the pipeline group by the stage that owns it (the first stage for a tied embedding).
    ``pp`` is the pipeline ``GroupInfo``. Returns the bytes received by this rank."""
    import torch.distributed as dist

    mine = torch.tensor(list(src_store.layer_range), device=dst_store.device)
    allr = [torch.empty_like(mine) for _ in range(pp.size)]
    dist.all_gather(allr, mine, group=pp.group)
    spans = [tuple(int(v) for v in t.tolist()) for t in allr]

    def owner(name: str) -> int:
        if name.startswith("layers."):
            i = int(name.split(".")[1])
            return next(r for r, (lo, hi) in enumerate(spans) if lo <= i < hi)
        return 0 if name == "embed.weight" else pp.size - 1

    moved = 0
    for s in dst_store.specs:
        o = owner(s.name)
        dst = dst_store.params[s.name]
        if o == pp.rank:
            dst.copy_(src_store.params[s.name].to(dst.dtype))
        else:
            moved += dst.numel() * dst.element_size()
        dist.broadcast(dst, src=pp.ranks[o], group=pp.group)
    return moved
