"""Partitioned optimizer for the replicated ("dense") parameters: gradient reduce-scatter, Adam on the owned range and
parameter all-gather as kernels over NVLink peer memory (``csrc/dp_adam.cu``), ZeRO-1 style.

The flat dense parameter buffer (bf16) and gradient buffer (fp32) are moved into a symmetric region that every
data-parallel rank maps. Rank ``r`` owns elements ``[lo, hi)`` and keeps moments (and the fp32 master copy) only for
them. A step is: signal "gradients final" / wait for all ranks -> every rank sums its range over all peers' gradient
buffers (P2P loads, fixed rank order) and produces the range's sum of squares -> global norm and clip coefficient on
the device -> Adam on the range, new bf16 parameters stored into every rank's parameter buffer (P2P stores) ->
signal "pushed" / wait. No NCCL call, no staging copy; the two waits are the only synchronisation.

Reference: Megatron's distributed optimizer (reduce-scatter + FusedAdam on the shard + all-gather), forced on for Adam
in miles/backends/megatron_utils/arguments.py:15-17.
"""
from __future__ import annotations

import torch

from ..ops import _ext
from .symm import SymmetricRegion


class ShardedDenseAdam:
    def __init__(self, store, group, rank: int, size: int, device: torch.device, cfg):
        assert size > 1 and device.type == "cuda"
        self.store, self.rank, self.n, self.dev, self.cfg = store, rank, size, device, cfg
        self.C = _ext.load(required=True)
        flat = store.flat["dense"]
        assert flat.dtype == torch.bfloat16, "the partitioned optimizer keeps bf16 parameters"
        N = flat.numel()
        per = (N + size - 1) // size
        per = (per + 127) // 128 * 128
        self.lo, self.hi = min(N, rank * per), min(N, rank * per + per)
        self.region = SymmetricRegion(N * 4 + N * 2 + 4 * size * 8 + 8192, group, rank, size, device)
        self.grad_sym, self.p_grad = self.region.carve((N,), torch.float32)
        self.param_sym, self.p_param = self.region.carve((N,), torch.bfloat16)
        self.flags, self.p_flags = self.region.carve((size,), torch.int64)
        self.flags2, self.p_flags2 = self.region.carve((size,), torch.int64)
        self._peers = (self.p_grad, self.p_param, self.p_flags, self.p_flags2)
        self.param_sym.copy_(flat)
        store.rebind_flat("dense", self.param_sym)
        store.pin_grad_storage("dense", self.grad_sym)
        n = self.hi - self.lo
        self.m = torch.zeros(n, dtype=cfg.state_dtype, device=device)
        self.v = torch.zeros(n, dtype=cfg.state_dtype, device=device)
        self.master = self.param_sym[self.lo:self.hi].float().clone() if cfg.master_weights else None
        self.reduced = torch.zeros(max(n, 8), dtype=torch.float32, device=device)[:n]
        self.ctrl = torch.zeros(8, dtype=torch.int64, device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self.bytes_read = self.bytes_pushed = 0

    def reduce(self) -> torch.Tensor:
        """Reduce-scatter: fills ``self.reduced`` with the summed gradients of the owned range; returns its sum of
        squares (a device scalar)."""
        C = self.C
        C.peer_signal(*self._peers, self.rank, self.ctrl, 0, False)
        C.ep_wait(self.flags, self.n, self.ctrl, 1, self.status)
        if self.hi <= self.lo:
            return torch.zeros((), dtype=torch.float32, device=self.dev)
        partial = C.dp_reduce_shard(*self._peers, self.lo, self.reduced)
        self.bytes_read += (self.n - 1) * (self.hi - self.lo) * 4
        return partial.sum()

    def apply(self, segments, lr: float, step: int, grad_scale: torch.Tensor, skip_flag: torch.Tensor) -> None:
        """Adam on the owned range (one launch per weight-decay segment that intersects it), parameters pushed to
        every rank; returns after all peers' pushes have landed here."""
        C, c = self.C, self.cfg
        for a, b, wd in segments:
            a, b = max(a, self.lo), min(b, self.hi)
            if b <= a:
                continue
            s = slice(a - self.lo, b - self.lo)
            C.dp_adam_push(*self._peers, self.rank, a, self.reduced[s], self.master[s] if self.master is not None else None,
                           self.m[s], self.v[s], lr, c.beta1, c.beta2, c.eps, wd, step, grad_scale, skip_flag)
            self.bytes_pushed += (self.n - 1) * (b - a) * 2
        C.peer_signal(*self._peers, self.rank, self.ctrl, 2, True)
        C.ep_wait(self.flags2, self.n, self.ctrl, 3, self.status)

    def check_status(self) -> None:
        code = int(self.status.item())
        if code:
            self.status.zero_()
            raise RuntimeError(f"partitioned optimizer exchange reported error {code} (5 = a peer never signalled)")

    def sync_master_from_params(self) -> None:
        if self.master is not None:
            self.master.copy_(self.param_sym[self.lo:self.hi].float())
