"""The device mesh of the sharded data-parallel backend: ``replicate x shard``.

Shard ranks are consecutive (the GPUs of one NVLink domain share a model copy), replicas stride over them, the layout of
``(dp_replicate, dp_shard)`` in the reference (miles/backends/fsdp_utils/parallel.py:14-103,
``validate_hybrid_shard_args`` in fsdp_utils/arguments.py:125-133).
"""
from __future__ import annotations

from dataclasses import dataclass

from ..parallel.reloadable_groups import registry
from ..parallel.state import GroupInfo, ParallelState


@dataclass
class FsdpMesh:
    shard: GroupInfo
    replicate: GroupInfo


def mesh_ranks(ranks: list, replicate_size: int) -> tuple:
    """``ranks``: the data-parallel ranks in order. Returns (shard groups, replicate groups) as lists of rank lists."""
    n = len(ranks)
    if replicate_size < 1 or n % replicate_size:
        raise ValueError(f"--dp-replicate-size {replicate_size} must divide the data-parallel size {n}")
    s = n // replicate_size
    shard = [ranks[i * s:(i + 1) * s] for i in range(replicate_size)]
    repl = [ranks[j::s] for j in range(s)]
    return shard, repl


def build_mesh(ps: ParallelState, replicate_size: int = 1) -> FsdpMesh:
    """Collective over all ranks of the job (every rank creates every group, in the same order)."""
    ranks = list(ps.dp_cp.ranks) if ps.dp_cp.size > 1 else [ps.rank]
    if len(ranks) == 1:
        return FsdpMesh(GroupInfo(0, 1, None, ranks), GroupInfo(0, 1, None, ranks))
    if replicate_size == 1:
        return FsdpMesh(GroupInfo(ps.dp_cp.rank, ps.dp_cp.size, ps.dp_cp.group, ranks), GroupInfo(0, 1, None, [ps.rank]))
    shard_groups, repl_groups = mesh_ranks(ranks, replicate_size)
    mine_s = mine_r = None
    for rk in shard_groups:
        g = registry().new_group(rk) if len(rk) > 1 else None
        if ps.rank in rk:
            mine_s = GroupInfo(rk.index(ps.rank), len(rk), g, rk)
    for rk in repl_groups:
        g = registry().new_group(rk) if len(rk) > 1 else None
        if ps.rank in rk:
            mine_r = GroupInfo(rk.index(ps.rank), len(rk), g, rk)
    return FsdpMesh(mine_s, mine_r)
