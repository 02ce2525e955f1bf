"""Tensor parallelism for the attention and dense-MLP projections.

Column-parallel projections (qkv, gate_up) need no communication in the forward pass and an all-reduce of the
input gradient in the backward pass; row-parallel projections (o, down) the reverse. Every all-reduced tensor
is ``[tokens, hidden]``.

Fused path: the row-parallel (or input-gradient) GEMM does not write its partial result locally at all. Its
epilogue stores each tile into slot ``rank`` of every rank's symmetric partial-sum buffer over NVLink (plain
16-byte peer stores of whole 256-byte row segments, issued tile by tile while later tiles are still being
multiplied), and the last CTA raises an arrival flag on every peer. The consumer waits for the flags of this
epoch and adds the slots in rank order (plus the residual), so all ranks obtain bit-identical sums, which is
what lets the replicated parts of the model, and the replicated rollout engines, stay in lockstep. Bytes sent
per rank are ``(tp - 1) * T * H * 2``: for TP2 the same as a ring all-reduce, above that the price of a
deterministic one-step exchange on an NVSwitch fabric that gives every pair full bandwidth.

Baseline path (``fused=False``): local GEMM + NCCL ``all_reduce``.

Reference: Megatron column/row-parallel linears driven by ``--tensor-model-parallel-size``
(miles/backends/megatron_utils/initialize.py:45-61); SP all-gather/reduce-scatter is folded into the same
exchange here because activations stay replicated between the two collectives of a layer.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from ..ops import _ext


class TensorParallel:
    def __init__(self, group, rank: int, size: int, device: torch.device, hidden: int, max_tokens: int, fused: bool = True):
        self.group, self.rank, self.n, self.dev = group, rank, size, device
        self.H, self.max_tokens = hidden, max_tokens
        self.fused = fused and device.type == "cuda" and size > 1
        self.C = _ext.load(required=True) if device.type == "cuda" else None
        self.bytes_sent = 0
        self._parity = 0
        if self.fused:
            from .symm import SymmetricRegion

            slot = max_tokens * hidden
            nbytes = 2 * size * slot * 2 + 4096
            self.region = SymmetricRegion(nbytes, group, rank, size, device)
            self.bufs, self.p_bufs = [], []
            for _ in range(2):  # two generations: a peer may still be adding up generation k while k+1 arrives
                t, p = self.region.carve((size, slot), torch.bfloat16)
                self.bufs.append(t)
                self.p_bufs.append(p)
            self.flags, self.p_flags = self.region.carve((size,), torch.int64)
            self.ctrl = torch.zeros(8, dtype=torch.int64, device=device)
            self.status = torch.zeros(1, dtype=torch.int32, device=device)
            self.slot_bytes = slot * 2

    def check_status(self) -> None:
        if self.fused:
            code = int(self.status.item())
            if code:
                self.status.zero_()
                raise RuntimeError(f"tensor-parallel exchange reported error {code} (5 = a peer's partial sums never arrived)")

    def linear_allreduce(self, a: torch.Tensor, w: torch.Tensor, b_mn: bool = False,
                         residual: Optional[torch.Tensor] = None, gemm_status: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``all_reduce(a @ w^T)`` (``b_mn``: ``a @ w``) over the tensor-parallel group, plus ``residual``."""
        T = a.shape[0]
        N = w.shape[1] if b_mn else w.shape[0]
        assert N == self.H and T <= self.max_tokens, (N, self.H, T, self.max_tokens)
        out = torch.empty(T, N, dtype=torch.bfloat16, device=a.device)
        if self.n == 1:
            self.C.gemm(a, w, out, False, b_mn, False, 0, gemm_status)
            return out if residual is None else out.add_(residual)
        if not self.fused:
            self.C.gemm(a, w, out, False, b_mn, False, 0, gemm_status)
            dist.all_reduce(out, group=self.group)
            return out if residual is None else out.add_(residual)
        g = self._parity
        self._parity ^= 1
        dest = [p + self.rank * self.slot_bytes for p in self.p_bufs[g]]
        local_slot = self.bufs[g][self.rank][:T * N].view(T, N)  # shape/stride carrier; the kernel writes through `dest`
        self.C.gemm(a, w, local_slot, False, b_mn, False, 0, gemm_status, dest, self.ctrl, self.p_flags, self.rank)
        self.C.ep_wait(self.flags, self.n, self.ctrl, 3, self.status)
        self.C.sum_slots(self.bufs[g], residual, out)
        self.bytes_sent += (self.n - 1) * T * N * 2
        return out

    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        """Plain all-reduce for the few tensors that do not come out of a GEMM."""
        if self.n > 1:
            dist.all_reduce(x, group=self.group)
        return x
