"""Independent data-parallel replicas ("cells") that can come and go between steps.

Every cell is a complete trainer world of its own (its own default process group, its own tp / pp / ep layout).
Cells average gradients through a *reconfigurable* cross-cell group that is rebuilt whenever the quorum changes:

* ``ReconfigurableGroup.configure(addr, port, quorum_id, rank, world)`` tears the previous group down and joins
  the group of the new quorum (a stand-alone rendezvous, independent of the cell's default group; rank ``r`` of
  every cell talks to rank ``r`` of the other cells).
* ``allreduce`` never raises: a failed or timed-out collective marks the group errored, the step's result is then
  discarded by ``should_commit`` — a consensus (MIN over the cells) so that either every cell applies the step or
  none does.
* ``send_checkpoint`` / ``recv_checkpoint`` stream a trainer's state (flat parameter buffers, optimizer state,
  step counters) from a surviving cell to a healed one over the same group; tensors that share storage are sent
  once.

Failures are detected on the host (timeouts, exceptions); nothing here faults a GPU.

Reference counterpart: miles/backends/megatron_utils/ft/indep_dp.py:24-185 and ft/checkpoint_transfer.py:24-106 (on
torchft process groups and its PGTransport).
"""
from __future__ import annotations

import io
import time
from typing import Optional, Sequence

import torch
import torch.distributed as dist

from ..weight_sync.broadcast import destroy_update_group, init_update_group


class ReconfigurableGroup:
    def __init__(self, backend: str = "gloo", timeout_s: float = 60.0, name: str = "cells"):
        self.backend, self.timeout_s, self.name = backend, timeout_s, name
        self.pg = None
        self.quorum_id: Optional[int] = None
        self.rank = self.world = 0
        self._error: Optional[BaseException] = None

    # ------------------------------------------------------------------ lifecycle
    def _group_name(self, quorum_id: int) -> str:
        return f"{self.name}-q{quorum_id}"

    def configure(self, master_address: str, master_port: int, quorum_id: int, rank: int, world: int) -> None:
        """Join the cross-cell group of quorum ``quorum_id`` as ``rank`` of ``world`` cells."""
        self.shutdown()
        self._error = None
        self.rank, self.world, self.quorum_id = rank, world, quorum_id
        if world > 1:
            self.pg = init_update_group(master_address, master_port, rank, world, self._group_name(quorum_id),
                                        backend=self.backend, timeout_s=self.timeout_s)

    def shutdown(self) -> None:
        if self.pg is not None and self.quorum_id is not None:
            destroy_update_group(self._group_name(self.quorum_id))
        self.pg = None

    # ------------------------------------------------------------------ collectives that report instead of raising
    def errored(self) -> Optional[BaseException]:
        return self._error

    def report_error(self, e: BaseException) -> None:
        if self._error is None:
            self._error = e

    def allreduce(self, tensors: Sequence[torch.Tensor], average: bool = True) -> None:
        if self.world <= 1 or self._error is not None:
            return
        try:
            works = [dist.all_reduce(t, group=self.pg, async_op=True) for t in tensors]
            for w in works:
                w.wait()
            if average:
                for t in tensors:
                    t.div_(self.world)
        except Exception as e:  # a peer died or the collective timed out: the step will be discarded
            self.report_error(e)

    def should_commit(self, local_ok: bool = True) -> bool:
        """True only if every cell finished the step without an error (consensus over the cells)."""
        ok = local_ok and self._error is None
        if self.world <= 1:
            return ok
        flag = torch.tensor([1.0 if ok else 0.0])
        try:
            dist.all_reduce(flag.to("cuda") if self.backend == "nccl" else flag, op=dist.ReduceOp.MIN, group=self.pg)
        except Exception as e:
            self.report_error(e)
            return False
        return bool(flag.item() > 0.5)

    # ------------------------------------------------------------------ in-memory checkpoint transfer
    def send_checkpoint(self, state: dict, dst: int) -> int:
        """Send ``state`` (nested dict of tensors and picklable leaves) to cell ``dst``. Returns the bytes sent."""
        meta, tensors = _flatten_state(state)
        buf = io.BytesIO()
        torch.save(meta, buf)
        raw = torch.frombuffer(bytearray(buf.getvalue()), dtype=torch.uint8)
        dev = "cuda" if self.backend == "nccl" else "cpu"
        dist.send(torch.tensor([raw.numel()], dtype=torch.int64, device=dev), dst, group=self.pg)
        dist.send(raw.to(dev), dst, group=self.pg)
        sent = raw.numel()
        for t in tensors:
            dist.send(t.detach().contiguous().to(dev), dst, group=self.pg)
            sent += t.numel() * t.element_size()
        return sent

    def recv_checkpoint(self, src: int) -> dict:
        dev = "cuda" if self.backend == "nccl" else "cpu"
        n = torch.zeros(1, dtype=torch.int64, device=dev)
        dist.recv(n, src, group=self.pg)
        raw = torch.empty(int(n.item()), dtype=torch.uint8, device=dev)
        dist.recv(raw, src, group=self.pg)
        meta = torch.load(io.BytesIO(raw.cpu().numpy().tobytes()), weights_only=False)
        tensors = []
        for shape, dtype in meta["tensors"]:
            t = torch.empty(shape, dtype=dtype, device=dev)
            dist.recv(t, src, group=self.pg)
            tensors.append(t)
        return _unflatten_state(meta, tensors)


def _flatten_state(state: dict) -> tuple:
    """(meta, tensors): tensors that share storage (same data pointer, shape, dtype) are listed once."""
    tensors: list = []
    seen: dict = {}

    def walk(x):
        if isinstance(x, torch.Tensor):
            key = (x.data_ptr(), tuple(x.shape), x.dtype, tuple(x.stride()))
            if key not in seen:
                seen[key] = len(tensors)
                tensors.append(x)
            return {"__tensor__": seen[key]}
        if isinstance(x, dict):
            return {k: walk(v) for k, v in x.items()}
        if isinstance(x, (list, tuple)):
            return [walk(v) for v in x]
        return x

    tree = walk(state)
    return {"tree": tree, "tensors": [(tuple(t.shape), t.dtype) for t in tensors]}, tensors


def _unflatten_state(meta: dict, tensors: list):
    def walk(x):
        if isinstance(x, dict):
            if set(x) == {"__tensor__"}:
                return tensors[x["__tensor__"]]
            return {k: walk(v) for k, v in x.items()}
        if isinstance(x, list):
            return [walk(v) for v in x]
        return x

    return walk(meta["tree"])


def trainer_state(actor) -> dict:
    """What a healed cell needs to continue exactly where the survivors are."""
    return {"flat": dict(actor.store.flat), "version": actor.store.version, "global_step": actor.global_step,
            "optimizer": actor.opt.state_dict() if actor.opt is not None else None}


@torch.no_grad()
def load_trainer_state(actor, state: dict) -> None:
    for g, t in actor.store.flat.items():
        t.copy_(state["flat"][g].to(t.device, t.dtype))
    actor.store.version = int(state["version"])
    actor.global_step = int(state["global_step"])
    if actor.opt is not None and state.get("optimizer") is not None:
        actor.opt.load_state_dict(state["optimizer"])


def cross_cell_grad_sync(actor, group: ReconfigurableGroup, loss: Optional[torch.Tensor] = None) -> bool:
    """After a cell's own backward (and its intra-cell reductions): average the gradient buffers over the cells and
    agree on whether the step counts. Returns False if the step must be discarded (the caller then skips
    ``optimizer.step`` and zeroes the gradients)."""
    t0 = time.perf_counter()
    bufs = [g for g in actor.store.grad.values() if g is not None and g.numel()]
    if loss is not None:
        bufs = bufs + [loss]
    # pre-flight consensus: a cell that failed on the host before this point still answers here (one small
    # all-reduce), so the others skip the large one instead of waiting for a partner that will not come
    ok = group.should_commit()
    if ok:
        group.allreduce(bufs, average=True)
        ok = group.should_commit()
    actor.last_cross_cell_sync_s = time.perf_counter() - t0
    return ok
