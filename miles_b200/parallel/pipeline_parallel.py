"""Pipeline parallelism: contiguous layer ranges per stage and the one-forward-one-backward (1F1B) schedule.

A stage owns layers ``[lo, hi)`` of the model (the first stage also the embedding, the last one the final norm and
the LM head). Micro-batches flow through the stages as ``[tokens, hidden]`` activations over ``torch.distributed``
point-to-point operations (NCCL on GPUs, gloo on CPU); every stage holds the micro-batch metadata (tokens,
positions, sequence boundaries), so shapes are known on both sides of a transfer and only activations travel.

The schedule is the non-interleaved 1F1B: stage ``s`` of ``P`` runs ``min(P - s - 1, M)`` warm-up forwards, then
alternates one forward and one backward, then drains the remaining backwards. A send that has a receive in the
opposite direction at the same point of the schedule is issued together with it (`batch_isend_irecv`), which is what
keeps neighbouring stages from blocking each other. The model code is passed in as two callables, so the same
schedule drives the sm_100a model, the PyTorch model and the toy stages of the CPU tests.

Reference counterpart: Megatron's `get_forward_backward_func()` pipeline schedules as used by
miles/backends/megatron_utils/model.py:365-381 (forward only) and :560-570 (training).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional, Sequence

import torch
import torch.distributed as dist


def stage_layers(num_layers: int, pp_size: int, pp_rank: int, first: Optional[int] = None, last: Optional[int] = None) -> tuple[int, int]:
    """Layer range ``[lo, hi)`` of a stage. Layers are split evenly, the remainder going to the earliest stages;
    ``first`` / ``last`` fix the layer counts of the first / last stage (uneven pipelines: the stages that also hold
    the embedding or the LM head can be given fewer layers)."""
    if pp_size <= 1:
        return 0, num_layers
    counts = [0] * pp_size
    rest, stages = num_layers, list(range(pp_size))
    if first is not None:
        counts[0] = first
        rest -= first
        stages.remove(0)
    if last is not None and pp_size > 1:
        counts[-1] = last
        rest -= last
        stages.remove(pp_size - 1)
    if rest < 0 or (not stages and rest != 0):
        raise ValueError("first/last stage layer counts do not fit the model")
    for j, s in enumerate(stages):
        counts[s] = rest // len(stages) + (1 if j < rest % len(stages) else 0)
    lo = sum(counts[:pp_rank])
    return lo, lo + counts[pp_rank]


@dataclass
class PipeGroup:
    group: Optional[dist.ProcessGroup]
    rank: int            # position in the pipeline
    size: int
    ranks: Sequence[int]  # global ranks of the stages, in pipeline order

    @property
    def is_first(self) -> bool:
        return self.rank == 0

    @property
    def is_last(self) -> bool:
        return self.rank == self.size - 1

    @property
    def prev(self) -> int:
        return self.ranks[self.rank - 1]

    @property
    def next(self) -> int:
        return self.ranks[self.rank + 1]


class PipelineSchedule:
    """Runs micro-batches through this rank's stage.

    ``act_meta(mb) -> (shape, dtype)`` of the activation that enters / leaves a stage for micro-batch ``mb``.
    ``forward(mb, x_in) -> x_out``: ``x_in`` is None on the first stage; the return value is ignored on the last.
    ``backward(mb, dx_out) -> dx_in``: ``dx_out`` is None on the last stage (it derives the gradient from its loss);
    the return value is ignored on the first stage.
    """

    def __init__(self, pg: PipeGroup, device: torch.device):
        self.pg = pg
        self.device = device
        self.log: list = []  # ("F" | "B", micro-batch) in execution order, for tests and debugging

    # -------------------------------------------------------------- transfers
    def _exchange(self, send: Optional[torch.Tensor], send_to: Optional[int], recv_meta, recv_from: Optional[int]) -> Optional[torch.Tensor]:
        ops, out = [], None
        if send is not None and send_to is not None:
            ops.append(dist.P2POp(dist.isend, send.contiguous(), send_to, self.pg.group))
        if recv_meta is not None and recv_from is not None:
            out = torch.empty(recv_meta[0], dtype=recv_meta[1], device=self.device)
            ops.append(dist.P2POp(dist.irecv, out, recv_from, self.pg.group))
        if ops:
            for w in dist.batch_isend_irecv(ops):
                w.wait()
        return out

    # -------------------------------------------------------------- schedules
    def run_forward_only(self, n_mb: int, act_meta: Callable, forward: Callable) -> None:
        pg = self.pg
        for mb in range(n_mb):
            x = None if pg.is_first else self._exchange(None, None, act_meta(mb), pg.prev)
            y = forward(mb, x)
            self.log.append(("F", mb))
            if not pg.is_last:
                self._exchange(y, pg.next, None, None)

    def run_1f1b(self, n_mb: int, act_meta: Callable, forward: Callable, backward: Callable) -> None:
        pg = self.pg
        warm = min(pg.size - pg.rank - 1, n_mb)
        steady = n_mb - warm
        x_in = None
        if not pg.is_first and n_mb > 0:
            x_in = self._exchange(None, None, act_meta(0), pg.prev)
        for mb in range(warm):
            y = forward(mb, x_in)
            self.log.append(("F", mb))
            # send this activation on; the next forward's input arrives in the same exchange when there is one
            more_fwd = mb + 1 < n_mb
            nxt = self._exchange(y if not pg.is_last else None, pg.next if not pg.is_last else None,
                                 act_meta(mb + 1) if (more_fwd and not pg.is_first and (mb + 1 < warm or steady > 0)) else None,
                                 pg.prev if not pg.is_first else None)
            x_in = nxt
        for j in range(steady):
            f, b = warm + j, j
            y = forward(f, x_in)
            self.log.append(("F", f))
            # forward output goes down, the gradient of the oldest outstanding micro-batch comes back
            dy = None
            if not pg.is_last:
                dy = self._exchange(y, pg.next, act_meta(b), pg.next)
            dx = backward(b, dy)
            self.log.append(("B", b))
            more_fwd = f + 1 < n_mb
            if not pg.is_first:
                x_in = self._exchange(dx, pg.prev, act_meta(f + 1) if more_fwd else None, pg.prev)
        for b in range(steady, n_mb):
            dy = None if pg.is_last else self._exchange(None, None, act_meta(b), pg.next)
            dx = backward(b, dy)
            self.log.append(("B", b))
            if not pg.is_first:
                self._exchange(dx, pg.prev, None, None)
