"""Muon: momentum orthogonalised by a Newton-Schulz iteration for the weight matrices, Adam for everything else.

For a matrix parameter ``W`` with gradient ``G``:  ``M <- mu * M + G``;  ``U = G + mu * M`` (Nesterov) or ``M``;
``O = NS(U)`` is the nearest semi-orthogonal matrix (all singular values pushed to ~1 by a quintic Newton-Schulz
iteration run in bf16); ``W <- W - lr * (scale * O + wd * W)`` with ``scale = sqrt(max(1, rows / cols))`` ("spectral")
or ``0.2 * sqrt(max(rows, cols))`` ("unit_rms_norm", the update then has the RMS of an Adam step). The fused q/k/v
projection is orthogonalised per q, k and v block (``split_qkv``), expert tensors ``[E, rows, cols]`` per expert in
one batched iteration. Embedding, LM head, router, norm weights and biases use Adam.

The class has the interface of ``FlatAdam`` (``step`` returns the pre-clip global gradient norm, ``state_dict`` /
``load_state_dict``, ``cfg``, ``step_count``) so the actor can hold either.

Reference counterpart: the Muon branch of the optimizer builder, miles/backends/megatron_utils/model.py:125-210
(``get_megatron_muon_optimizer``, ``muon_split_qkv``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist

from ..models.params import ParamStore
from .optimizer import OptimConfig, lr_at

NS_COEFFS = (3.4445, -4.7750, 2.0315)


@dataclass
class MuonConfig:
    momentum: float = 0.95
    nesterov: bool = True
    ns_steps: int = 5
    scale_mode: str = "spectral"   # "spectral" | "unit_rms_norm"
    extra_scale: float = 1.0
    split_qkv: bool = True


@torch.no_grad()
def newton_schulz(G: torch.Tensor, steps: int = 5, eps: float = 1e-7) -> torch.Tensor:
    """Quintic Newton-Schulz iteration on the last two dimensions of ``G`` (batched over the leading ones)."""
    a, b, c = NS_COEFFS
    X = G.to(torch.bfloat16 if G.is_cuda else torch.float32)
    transposed = X.shape[-2] > X.shape[-1]
    if transposed:
        X = X.transpose(-2, -1)
    X = X / (X.float().norm(dim=(-2, -1), keepdim=True).to(X.dtype) + eps)
    for _ in range(steps):
        A = X @ X.transpose(-2, -1)
        B = b * A + c * (A @ A)
        X = a * X + B @ X
    if transposed:
        X = X.transpose(-2, -1)
    return X


def is_muon_param(name: str, shape: tuple) -> bool:
    if len(shape) < 2 or name in ("embed.weight", "lm_head.weight") or name.endswith("moe.router.weight"):
        return False
    return name.endswith((".weight", "moe.w1", "moe.w2"))


class Muon:
    def __init__(self, store: ParamStore, cfg: OptimConfig, mcfg: Optional[MuonConfig] = None, dp_group=None, ep_group=None,
                 tp_group=None, pp_group=None):
        self.store, self.cfg, self.mcfg = store, cfg, mcfg or MuonConfig()
        self.ep_group, self.pp_group, self.tp_group = ep_group, pp_group, tp_group
        self.dev = store.device
        self.step_count = 0
        self.launches = 0
        self.h2d_bytes = self.d2h_bytes = 0
        self.last_grad_norm: Optional[torch.Tensor] = None
        self.muon_names = [n for n, p in store.params.items() if is_muon_param(n, tuple(p.shape))]
        self.adam_names = [n for n in store.params if n not in set(self.muon_names)]
        self.momentum = {n: torch.zeros_like(store.params[n], dtype=torch.float32) for n in self.muon_names}
        self.exp_avg = {n: torch.zeros_like(store.params[n], dtype=torch.float32) for n in self.adam_names}
        self.exp_avg_sq = {n: torch.zeros_like(store.params[n], dtype=torch.float32) for n in self.adam_names}
        # fp32 master copies keep updates smaller than a bf16 ulp from being lost
        self.master = {n: p.detach().float().clone() for n, p in store.params.items()} if (cfg.master_weights and store.dtype != torch.float32) else None

    # ------------------------------------------------------------------ norm / clip
    @torch.no_grad()
    def compute_grad_norm(self) -> torch.Tensor:
        buf = torch.zeros(2, dtype=torch.float32, device=self.dev)
        for i, g in enumerate(("dense", "expert")):
            gr = self.store.grad.get(g)
            if gr is not None and gr.numel():
                buf[i] = gr.float().pow(2).sum()
        if dist.is_available() and dist.is_initialized():
            if self.ep_group is not None and dist.get_world_size(self.ep_group) > 1:
                dist.all_reduce(buf[1:2], group=self.ep_group)
            if self.pp_group is not None and dist.get_world_size(self.pp_group) > 1:
                dist.all_reduce(buf, group=self.pp_group)
        self.last_grad_norm = buf.sum().sqrt()
        return self.last_grad_norm

    def _scale(self, rows: int, cols: int) -> float:
        m = self.mcfg
        s = max(1.0, rows / cols) ** 0.5 if m.scale_mode == "spectral" else 0.2 * max(rows, cols) ** 0.5
        return s * m.extra_scale

    def _orthogonalise(self, name: str, U: torch.Tensor) -> torch.Tensor:
        m = self.mcfg
        if name.endswith("attn.qkv.weight") and m.split_qkv:
            q, kv = self.store.cfg.q_dim, self.store.cfg.kv_dim
            parts = [U[:q], U[q:q + kv], U[q + kv:]]
            return torch.cat([newton_schulz(p, m.ns_steps).float() * self._scale(*p.shape[-2:]) for p in parts], 0)
        return newton_schulz(U, m.ns_steps).float() * self._scale(*U.shape[-2:])

    # ------------------------------------------------------------------ step
    @torch.no_grad()
    def step(self, grad_scale: float = 1.0) -> torch.Tensor:
        c, m = self.cfg, self.mcfg
        norm = self.compute_grad_norm()
        coef = torch.ones((), device=self.dev)
        if c.clip_grad and c.clip_grad > 0:
            coef = torch.clamp(c.clip_grad / (norm * grad_scale + 1e-6), max=1.0)
        finite = torch.isfinite(norm)
        gs = coef * grad_scale
        lr = lr_at(c, self.step_count)
        self.step_count += 1
        if not bool(finite):
            return norm * grad_scale  # skipped step: a non-finite gradient leaves weights and state untouched
        t = self.step_count
        bc1, bc2 = 1.0 - c.beta1 ** t, 1.0 - c.beta2 ** t
        P, G = self.store.params, self.store.grads
        for n in self.muon_names:
            g = G[n].float() * gs
            M = self.momentum[n]
            M.mul_(m.momentum).add_(g)
            U = g.add(M, alpha=m.momentum) if m.nesterov else M
            upd = self._orthogonalise(n, U)
            w = self.master[n] if self.master is not None else P[n]
            w.mul_(1.0 - lr * c.weight_decay).add_(upd.to(w.dtype), alpha=-lr)
            if self.master is not None:
                P[n].copy_(w)
        for n in self.adam_names:
            g = G[n].float() * gs
            ea, es = self.exp_avg[n], self.exp_avg_sq[n]
            ea.mul_(c.beta1).add_(g, alpha=1.0 - c.beta1)
            es.mul_(c.beta2).addcmul_(g, g, value=1.0 - c.beta2)
            w = self.master[n] if self.master is not None else P[n]
            wd = c.weight_decay if w.dim() >= 2 else 0.0
            upd = (ea / bc1) / ((es / bc2).sqrt() + c.eps)
            w.mul_(1.0 - lr * wd).add_(upd.to(w.dtype), alpha=-lr)
            if self.master is not None:
                P[n].copy_(w)
        self.store.version += 1
        return norm * grad_scale

    # ------------------------------------------------------------------ state
    def promote_offloaded(self, max_bytes: int) -> int:
        return 0

    def state_dict(self) -> dict:
        cpu = lambda d: {k: v.cpu() for k, v in d.items()}
        return {"kind": "muon", "step": self.step_count, "momentum": cpu(self.momentum), "exp_avg": cpu(self.exp_avg),
                "exp_avg_sq": cpu(self.exp_avg_sq), "master": cpu(self.master) if self.master is not None else None}

    def load_state_dict(self, sd: dict) -> None:
        self.step_count = int(sd["step"])
        for mine, theirs in ((self.momentum, sd["momentum"]), (self.exp_avg, sd["exp_avg"]), (self.exp_avg_sq, sd["exp_avg_sq"])):
            for k, v in theirs.items():
                mine[k].copy_(v)
        if self.master is not None and sd.get("master") is not None:
            for k, v in sd["master"].items():
                self.master[k].copy_(v)

    def sync_master_from_params(self) -> None:
        if self.master is not None:
            for n, p in self.store.params.items():
                self.master[n].copy_(p)
