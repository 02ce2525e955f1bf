"""LoRA on the flat parameter store, in merged form.

Adapters ``A [r, in]`` / ``B [out, r]`` are kept in fp32 per target projection (HF/PEFT module names
``q_proj, k_proj, v_proj, o_proj, gate_proj, up_proj, down_proj``; fused native tensors are addressed by
row slices).  Before every forward the effective weight ``W = W_base + (alpha/r) * B @ A`` is written into
the store, so every kernel (trainer and the colocated engine, which shares the memory) runs unchanged
and the trainer -> rollout adapter sync is free.  Gradients follow from the full weight gradient the
GEMM epilogues already accumulate: ``dB = s * dW @ A^T``, ``dA = s * B^T @ dW``; only the adapters have
optimizer state.  Adapters are saved / loaded in PEFT layout (``adapter_model.safetensors`` +
``adapter_config.json``).

Reference: miles/backends/megatron_utils/lora_utils.py:113-647 (attach, name mapping, adapter-only
checkpoints) and update_weight_from_tensor.py:284-312 (adapter sync).
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from .models.params import ParamStore, _seed_for

ALL_LINEAR = ["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"]


@dataclass
class Target:
    hf_module: str       # e.g. model.layers.3.self_attn.q_proj
    native: str          # native tensor name
    row0: int
    row1: int
    expert: Optional[int] = None
    tp: Optional[str] = None   # under tensor parallelism: "col" (output rows sharded, A replicated), "row" (input columns
                               # sharded, B replicated), None (not sharded: experts)


def _targets(store: ParamStore, modules: Sequence[str]) -> list:
    cfg = store.cfg
    out = []
    q, kv = cfg.q_dim, cfg.kv_dim
    for i in range(*getattr(store, "layer_range", (0, cfg.num_layers))):
        p, hp = f"layers.{i}.", f"model.layers.{i}."
        att = {"q_proj": (0, q), "k_proj": (q, q + kv), "v_proj": (q + kv, q + 2 * kv)}
        for m, (a, b) in att.items():
            if m in modules:
                out.append(Target(hp + "self_attn." + m, p + "attn.qkv.weight", a, b, tp="col"))
        if "o_proj" in modules:
            out.append(Target(hp + "self_attn.o_proj", p + "attn.o.weight", 0, cfg.hidden_size, tp="row"))
        if not cfg.layer_is_moe(i):
            I = cfg.ffn_hidden_size
            if "gate_proj" in modules:
                out.append(Target(hp + "mlp.gate_proj", p + "mlp.gate_up.weight", 0, I, tp="col"))
            if "up_proj" in modules:
                out.append(Target(hp + "mlp.up_proj", p + "mlp.gate_up.weight", I, 2 * I, tp="col"))
            if "down_proj" in modules:
                out.append(Target(hp + "mlp.down_proj", p + "mlp.down.weight", 0, cfg.hidden_size, tp="row"))
        else:
            I = cfg.moe_ffn_hidden_size
            el = cfg.num_experts // store.ep_size
            for le in range(el):
                ge = store.ep_rank * el + le
                ep = hp + f"mlp.experts.{ge}."
                if "gate_proj" in modules:
                    out.append(Target(ep + "gate_proj", p + "moe.w1", 0, I, le))
                if "up_proj" in modules:
                    out.append(Target(ep + "up_proj", p + "moe.w1", I, 2 * I, le))
                if "down_proj" in modules:
                    out.append(Target(ep + "down_proj", p + "moe.w2", 0, cfg.hidden_size, le))
    return out


class LoRAManager:
    """``tp_group``: the tensor-parallel group of a store that holds a shard (``store.tp_size > 1``). The adapter of a
    column-parallel projection shards ``B`` by output rows and keeps ``A`` whole on every rank; a row-parallel one shards
    ``A`` by input columns and keeps ``B`` whole. The whole factor's gradient is a partial sum on each rank and is
    all-reduced over the group before the step, so the ranks stay equal and the sharded adapter is the unsharded one
    (the role of the partial-gradient all-reduce in miles/backends/megatron_utils/lora_utils.py)."""

    def __init__(self, store: ParamStore, rank: int, alpha: float, target_modules: Sequence[str] | str = "all-linear",
                 lr: float = 1e-4, weight_decay: float = 0.0, seed: int = 0, betas=(0.9, 0.999), base: Optional[dict] = None,
                 tp_group=None):
        assert rank > 0
        mods = ALL_LINEAR if target_modules in ("all-linear", None) else list(target_modules)
        self.store, self.rank, self.alpha = store, rank, float(alpha)
        self.scale = self.alpha / rank
        self.target_modules = mods
        self.targets = _targets(store, mods)
        self.tp_size, self.tp_rank = getattr(store, "tp_size", 1), getattr(store, "tp_rank", 0)
        self.tp_group = tp_group
        assert self.tp_size == 1 or tp_group is not None, "a tensor-parallel store needs the tensor-parallel group"
        dev = store.device
        self.A, self.B = [], []
        for t in self.targets:
            w = self._slice(store.params[t.native], t)
            # one generator per module, drawn at the unsharded width: the start does not depend on the layout
            g = torch.Generator(device="cpu").manual_seed(_seed_for(seed, t.hf_module))
            cols = w.shape[1] * (self.tp_size if t.tp == "row" else 1)
            a = torch.empty(rank, cols).uniform_(-1, 1, generator=g) * math.sqrt(3.0 / cols)
            if t.tp == "row" and self.tp_size > 1:
                a = a[:, self.tp_rank * w.shape[1]:(self.tp_rank + 1) * w.shape[1]].contiguous()
            self.A.append(a.to(dev).requires_grad_(False))
            self.B.append(torch.zeros(w.shape[0], rank, device=dev))
        # the factors every tensor-parallel rank holds whole (partial gradients) and the ones it holds a shard of
        self._whole = [] if self.tp_size == 1 else [a if t.tp == "col" else b for t, a, b in zip(self.targets, self.A, self.B) if t.tp]
        self._sharded = [] if self.tp_size == 1 else [b if t.tp == "col" else a for t, a, b in zip(self.targets, self.A, self.B) if t.tp]
        # frozen base copies of the targeted tensors only (several adapters on one model share one set: ``base``)
        need = {t.native for t in self.targets}
        self.base = base if base is not None else {}
        for n in need:
            if n not in self.base:
                self.base[n] = store.params[n].detach().clone()
        self.opt = torch.optim.AdamW([p for p in self.A + self.B], lr=lr, weight_decay=weight_decay, betas=betas)
        for p in self.A + self.B:
            p.grad = torch.zeros_like(p)


    @staticmethod
    def _slice(w: torch.Tensor, t: Target) -> torch.Tensor:
        if t.expert is not None:
            w = w[t.expert]
        return w[t.row0:t.row1]

    def num_parameters(self) -> int:
        return sum(p.numel() for p in self.A + self.B)

    @torch.no_grad()
    def merge(self) -> None:
        """Write ``base + scale * B @ A`` into the live weights."""
        for n, b in self.base.items():
            self.store.params[n].copy_(b)
        for t, a, b in zip(self.targets, self.A, self.B):
            w = self._slice(self.store.params[t.native], t)
            w.add_((self.scale * (b @ a)).to(w.dtype))

    @torch.no_grad()
    def check_merged(self, params: Optional[dict] = None, atol: float = 2e-2) -> None:
        """``--check-lora-weight-equal``: every targeted weight the rollout engine serves (``params``, default the
        trainer's own live weights) must equal ``base + scale * B @ A`` of the adapter just trained (up to the
        rounding of the weight dtype); a missing tensor or a mismatch raises."""
        params = params if params is not None else self.store.params
        want = {n: b.detach().float().clone() for n, b in self.base.items()}
        for t, a, b in zip(self.targets, self.A, self.B):
            self._slice(want[t.native], t).add_(self.scale * (b @ a))
        for n, w in want.items():
            if n not in params:
                raise AssertionError(f"adapter sync check: the engine has no tensor {n}")
            got = params[n].detach().float()
            err = (got - w.to(got.device)).abs().max().item()
            tol = atol * max(w.abs().max().item(), 1e-6)
            assert err <= tol, f"adapter sync check: {n} differs from base + scale*B@A by {err} (tolerance {tol})"

    @torch.no_grad()
    def grads_from_weight_grads(self) -> None:
        """Project the full weight gradients (already accumulated by the backward GEMMs) onto the adapters."""
        if self.tp_size > 1:
            part = torch.zeros(sum(p.numel() for p in self._whole), device=self.store.device)
            views, o = {}, 0
            for p in self._whole:
                views[id(p)] = part[o:o + p.numel()].view_as(p)
                o += p.numel()
        for t, a, b in zip(self.targets, self.A, self.B):
            dw = self._slice(self.store.grads[t.native], t).float()
            db, da = self.scale * (dw @ a.t()), self.scale * (b.t() @ dw)
            if self.tp_size > 1 and t.tp == "col":
                b.grad.add_(db)
                views[id(a)].copy_(da)
            elif self.tp_size > 1 and t.tp == "row":
                a.grad.add_(da)
                views[id(b)].copy_(db)
            else:
                b.grad.add_(db)
                a.grad.add_(da)
        if self.tp_size > 1 and part.numel():
            import torch.distributed as dist

            dist.all_reduce(part, group=self.tp_group)      # one collective for all partial gradients of the step
            for p in self._whole:
                p.grad.add_(views[id(p)])

    def grad_norm(self) -> torch.Tensor:
        if self.tp_size == 1:
            return torch.sqrt(sum((p.grad.float() ** 2).sum() for p in self.A + self.B))
        import torch.distributed as dist

        sharded = {id(p) for p in self._sharded}
        sq = sum((p.grad.float() ** 2).sum() for p in self.A + self.B if id(p) in sharded)
        sq = sq if torch.is_tensor(sq) else torch.zeros((), device=self.store.device)
        dist.all_reduce(sq, group=self.tp_group)            # shards add up over the group, whole factors count once
        return torch.sqrt(sq + sum((p.grad.float() ** 2).sum() for p in self.A + self.B if id(p) not in sharded))

    @torch.no_grad()
    def step(self, clip_grad: float = 0.0, grad_scale: float = 1.0) -> torch.Tensor:
        for p in self.A + self.B:
            p.grad.mul_(grad_scale)
        norm = self.grad_norm()
        if clip_grad and clip_grad > 0:
            coef = torch.clamp(clip_grad / (norm + 1e-6), max=1.0)
            for p in self.A + self.B:
                p.grad.mul_(coef)
        self.opt.step()
        for p in self.A + self.B:
            p.grad.zero_()
        self.merge()
        self.store.version += 1
        return norm

    # ------------------------------------------------------------------ PEFT checkpoint
    @torch.no_grad()
    def state_dict(self) -> dict:
        """PEFT-named tensors of the whole adapter. Under tensor parallelism the shards are gathered over the group (a
        collective: every rank of the group calls it) and every rank returns the unsharded adapter."""
        out = {}
        for t, a, b in zip(self.targets, self.A, self.B):
            a, b = a.detach(), b.detach()
            if self.tp_size > 1 and t.tp:
                import torch.distributed as dist

                mine = (b if t.tp == "col" else a).contiguous()
                parts = [torch.empty_like(mine) for _ in range(self.tp_size)]
                dist.all_gather(parts, mine, group=self.tp_group)
                a, b = (a, torch.cat(parts, 0)) if t.tp == "col" else (torch.cat(parts, 1), b)
            out[f"base_model.model.{t.hf_module}.lora_A.weight"] = a.cpu().contiguous()
            out[f"base_model.model.{t.hf_module}.lora_B.weight"] = b.cpu().contiguous()
        return out

    def _state_file(self) -> str:
        return "training_state.pt" if self.tp_size == 1 else f"training_state_tp{self.tp_rank}.pt"

    def save(self, path: str, base_model_name: str = "", write_adapter: bool = True) -> None:
        """Every rank of a tensor-parallel group calls it (the gather is collective); the rank with ``write_adapter``
        writes the PEFT files, every rank writes the optimizer state of its own shard."""
        from safetensors.torch import save_file

        sd = self.state_dict()
        os.makedirs(path, exist_ok=True)
        if write_adapter:
            save_file(sd, os.path.join(path, "adapter_model.safetensors"), metadata={"format": "pt"})
            cfg = {"peft_type": "LORA", "r": self.rank, "lora_alpha": self.alpha, "lora_dropout": 0.0, "bias": "none",
                   "target_modules": self.target_modules, "task_type": "CAUSAL_LM", "base_model_name_or_path": base_model_name}
            with open(os.path.join(path, "adapter_config.json"), "w") as f:
                json.dump(cfg, f, indent=1)
        torch.save({"optimizer": self.opt.state_dict()}, os.path.join(path, self._state_file()))

    def load(self, path: str, load_optimizer: bool = True) -> None:
        from safetensors.torch import load_file

        sd = load_file(os.path.join(path, "adapter_model.safetensors"))
        with torch.no_grad():
            for t, a, b in zip(self.targets, self.A, self.B):
                ka = f"base_model.model.{t.hf_module}.lora_A.weight"
                if ka in sd:
                    fa, fb = sd[ka], sd[ka.replace("lora_A", "lora_B")]
                    if self.tp_size > 1 and t.tp == "col":
                        fb = fb[self.tp_rank * b.shape[0]:(self.tp_rank + 1) * b.shape[0]]
                    elif self.tp_size > 1 and t.tp == "row":
                        fa = fa[:, self.tp_rank * a.shape[1]:(self.tp_rank + 1) * a.shape[1]]
                    a.copy_(fa)
                    b.copy_(fb)
        ts = os.path.join(path, self._state_file())
        if load_optimizer and os.path.exists(ts):
            self.opt.load_state_dict(torch.load(ts, weights_only=False)["optimizer"])
        self.merge()

    def adapter_tensors(self):
        """(hf name, tensor) pairs of the adapter only — what an external engine would load."""
        return list(self.state_dict().items())


@torch.no_grad()
def merge_adapter_into(store: ParamStore, tensors: dict, scale: float = 1.0) -> int:
    """Add ``scale * B @ A`` of a PEFT-named adapter (``...<module>.lora_A.weight`` / ``lora_B.weight``) into the
    weights of ``store``; a negative ``scale`` takes the same adapter out again. Returns the number of modules merged.
    Engines use it to serve an adapter without a second set of GEMMs."""
    by_module = {t.hf_module: t for t in _targets(store, ALL_LINEAR)}
    n = 0
    for key, a in tensors.items():
        if not key.endswith("lora_A.weight"):
            continue
        mod = key[:-len(".lora_A.weight")]
        mod = mod[len("base_model.model."):] if mod.startswith("base_model.model.") else mod
        b = tensors.get(key.replace("lora_A.weight", "lora_B.weight"))
        t = by_module.get(mod)
        if b is None or t is None:
            continue
        w = LoRAManager._slice(store.params[t.native], t)
        w.add_((scale * (b.to(w.device).float() @ a.to(w.device).float())).to(w.dtype))
        n += 1
    return n
