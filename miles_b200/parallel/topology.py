"""Which ranks share a node.

The peer-memory kernels of this package (expert dispatch / return, the tensor-parallel reduce, the partitioned optimizer,
the weight push, the low-latency decode exchange) address other GPUs through CUDA-IPC mappings, which exist only between
processes of one node. A group that spans nodes therefore takes the NCCL form of the same operation (the path
``--no-fused-comm`` selects everywhere), while groups inside a node keep the kernels. The usual multi-node layout then
works as it should: tensor / expert parallel groups inside the NVLink domain on peer memory, data parallelism across
nodes on NCCL.

A node is identified by its host name and boot id (two containers on one host have different host names but one
boot id and one set of GPUs; two hosts may carry the same container name).
"""
from __future__ import annotations

import os
import socket
from typing import Optional

import torch.distributed as dist

_cache: dict = {}


def node_identity() -> str:
    override = os.environ.get("MILES_B200_NODE_ID")  # tests, and schedulers that know better
    if override:
        return override
    boot = ""
    try:
        with open("/proc/sys/kernel/random/boot_id") as f:
            boot = f.read().strip()
    except OSError:
        pass
    return f"{socket.gethostname()}|{boot}"


def group_is_single_node(group=None, size: Optional[int] = None) -> bool:
    """Collective over ``group`` the first time it is asked about (every member must ask); cached afterwards."""
    if not (dist.is_available() and dist.is_initialized()):
        return True
    n = size if size is not None else dist.get_world_size(group)
    if n <= 1:
        return True
    key = id(group) if group is not None else 0
    if key not in _cache:
        ids = [None] * n
        dist.all_gather_object(ids, node_identity(), group=group)
        _cache[key] = len(set(ids)) == 1
    return _cache[key]


def peer_memory_ok(group=None, size: Optional[int] = None, wanted: bool = True) -> bool:
    """``wanted`` (the user's ``--fused-comm``) and every rank of the group on this node."""
    return bool(wanted) and group_is_single_node(group, size)
