"""Process groups of one training job.

Rank order is ``tp`` fastest, then ``cp``, ``ep``-within-``dp``, ``dp``, ``pp`` slowest (the
"tp-cp-ep-dp-pp" order the reference passes to Megatron, miles/backends/megatron_utils/initialize.py:41-61).
Expert parallelism reuses data-parallel ranks: the ``ep`` group is a contiguous slice of the ``dp x cp``
ranks, and the experts' own data-parallel group ("expert-dp") is what is left of dp after ep.

``ParallelState`` mirrors the fields of miles/backends/training_utils/parallel.py:32-79 (one ``GroupInfo``
per axis) so that the backend-agnostic training utilities can be written against it.  One process drives
one GPU; on a CPU box the same code runs over gloo.
"""
from __future__ import annotations

import datetime
import os
from dataclasses import dataclass, field
from typing import Optional

import torch
import torch.distributed as dist

from .reloadable_groups import registry, reset_registry


@dataclass
class GroupInfo:
    rank: int = 0
    size: int = 1
    group: Optional["dist.ProcessGroup"] = None
    ranks: list = field(default_factory=lambda: [0])

    @property
    def src_rank(self) -> int:
        return self.ranks[0]


@dataclass
class ParallelState:
    rank: int = 0
    world_size: int = 1
    local_rank: int = 0
    device: torch.device = torch.device("cpu")
    backend: str = "gloo"
    dp: GroupInfo = field(default_factory=GroupInfo)
    tp: GroupInfo = field(default_factory=GroupInfo)
    cp: GroupInfo = field(default_factory=GroupInfo)
    pp: GroupInfo = field(default_factory=GroupInfo)
    ep: GroupInfo = field(default_factory=GroupInfo)
    expert_dp: GroupInfo = field(default_factory=GroupInfo)
    dp_cp: GroupInfo = field(default_factory=GroupInfo)
    gloo_world: Optional["dist.ProcessGroup"] = None
    cp_comm_type: str = "p2p"

    @property
    def is_dp_src(self) -> bool:
        return self.tp.rank == 0 and self.cp.rank == 0 and self.pp.rank == self.pp.size - 1

    @property
    def effective_dp(self) -> GroupInfo:
        return self.dp


_STATE: Optional[ParallelState] = None


def get_parallel_state() -> ParallelState:
    global _STATE
    if _STATE is None:
        _STATE = ParallelState()
    return _STATE


def _make_groups(world: int, rank: int, layout: list, backend_timeout) -> dict:
    """``layout`` = [(name, size)] fastest-varying first; returns name -> GroupInfo for this rank."""
    import itertools

    sizes = [s for _, s in layout]
    assert torch.tensor(sizes).prod().item() == world, f"axis sizes {layout} do not multiply to world size {world}"
    strides, acc = [], 1
    for s in sizes:
        strides.append(acc)
        acc *= s
    out = {}
    for ai, (name, size) in enumerate(layout):
        others = [range(s) for j, s in enumerate(sizes) if j != ai]
        mine = None
        for combo in itertools.product(*others):
            base, k = 0, 0
            for j in range(len(sizes)):
                if j == ai:
                    continue
                base += combo[k] * strides[j]
                k += 1
            ranks = [base + i * strides[ai] for i in range(size)]
            grp = registry().new_group(ranks, timeout=backend_timeout) if size > 1 else None
            if rank in ranks:
                mine = GroupInfo(ranks.index(rank), size, grp, ranks)
        out[name] = mine
    return out


def init_parallel_state(tp: int = 1, pp: int = 1, cp: int = 1, ep: int = 1, backend: Optional[str] = None,
                        timeout_minutes: int = 10, cp_comm_type: str = "p2p") -> ParallelState:
    """Initialise torch.distributed from the torchrun environment (if needed) and build all axis groups."""
    global _STATE
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    cuda = torch.cuda.is_available()
    if backend is None:
        backend = "nccl" if cuda else "gloo"
    device = torch.device("cuda", local_rank) if cuda else torch.device("cpu")
    if cuda:
        torch.cuda.set_device(device)
    timeout = datetime.timedelta(minutes=timeout_minutes)
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        kw = {"device_id": device} if backend == "nccl" else {}
        dist.init_process_group(backend=backend, rank=rank, world_size=world, timeout=timeout, **kw)
    st = ParallelState(rank=rank, world_size=world, local_rank=local_rank, device=device, backend=backend,
                       cp_comm_type=cp_comm_type)
    if world > 1:
        assert world % (tp * pp * cp) == 0
        dp = world // (tp * pp * cp)
        assert (dp * cp) % ep == 0 or ep == 1, f"expert parallel size {ep} must divide dp*cp = {dp * cp}"
        g = _make_groups(world, rank, [("tp", tp), ("cp", cp), ("dp", dp), ("pp", pp)], timeout)
        st.tp, st.cp, st.dp, st.pp = g["tp"], g["cp"], g["dp"], g["pp"]
        # dp x cp combined (gradient reduction group of dense parameters)
        g2 = _make_groups(world, rank, [("tp", tp), ("dp_cp", dp * cp), ("pp", pp)], timeout)
        st.dp_cp = g2["dp_cp"]
        # experts: ep is a contiguous slice of dp_cp, expert_dp strides over it
        if ep > 1:
            g3 = _make_groups(world, rank, [("tp", tp), ("ep", ep), ("expert_dp", dp * cp // ep), ("pp", pp)], timeout)
            st.ep, st.expert_dp = g3["ep"], g3["expert_dp"]
        else:
            st.expert_dp = st.dp_cp
        if backend != "gloo":
            st.gloo_world = dist.new_group(list(range(world)), backend="gloo", timeout=timeout)
    _STATE = st
    return st


def destroy_parallel_state() -> None:
    global _STATE
    if dist.is_initialized():
        dist.destroy_process_group()
    reset_registry()
    _STATE = None
