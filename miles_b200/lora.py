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

from .models.params import ParamStore

ALL_LINEAR = ["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"]


@dataclass
class Target:
    hf_module: str       # e.g. model.layers.3.self_attn.q_proj
    native: str          # native tensor name
    row0: int
    row1: int
    expert: Optional[int] = None


def _targets(store: ParamStore, modules: Sequence[str]) -> list:
    cfg = store.cfg
    out = []
    q, kv = cfg.q_dim, cfg.kv_dim
    for i in range(*getattr(store, "layer_range", (0, cfg.num_layers))):
        p, hp = f"layers.{i}.", f"model.layers.{i}."
        att = {"q_proj": (0, q), "k_proj": (q, q + kv), "v_proj": (q + kv, q + 2 * kv)}
        for m, (a, b) in att.items():
            if m in modules:
                out.append(Target(hp + "self_attn." + m, p + "attn.qkv.weight", a, b))
        if "o_proj" in modules:
            out.append(Target(hp + "self_attn.o_proj", p + "attn.o.weight", 0, cfg.hidden_size))
        if not cfg.layer_is_moe(i):
            I = cfg.ffn_hidden_size
            if "gate_proj" in modules:
                out.append(Target(hp + "mlp.gate_proj", p + "mlp.gate_up.weight", 0, I))
            if "up_proj" in modules:
                out.append(Target(hp + "mlp.up_proj", p + "mlp.gate_up.weight", I, 2 * I))
            if "down_proj" in modules:
                out.append(Target(hp + "mlp.down_proj", p + "mlp.down.weight", 0, cfg.hidden_size))
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
    def __init__(self, store: ParamStore, rank: int, alpha: float, target_modules: Sequence[str] | str = "all-linear",
                 lr: float = 1e-4, weight_decay: float = 0.0, seed: int = 0, betas=(0.9, 0.999), base: Optional[dict] = None):
        assert rank > 0
        mods = ALL_LINEAR if target_modules in ("all-linear", None) else list(target_modules)
        self.store, self.rank, self.alpha = store, rank, float(alpha)
        self.scale = self.alpha / rank
        self.target_modules = mods
        self.targets = _targets(store, mods)
        dev = store.device
        g = torch.Generator(device="cpu").manual_seed(seed)
        self.A, self.B = [], []
        for t in self.targets:
            w = self._slice(store.params[t.native], t)
            a = torch.empty(rank, w.shape[1]).uniform_(-1, 1, generator=g) * math.sqrt(3.0 / w.shape[1])
            self.A.append(a.to(dev).requires_grad_(False))
            self.B.append(torch.zeros(w.shape[0], rank, device=dev))
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
        for t, a, b in zip(self.targets, self.A, self.B):
            dw = self._slice(self.store.grads[t.native], t).float()
            b.grad.add_(self.scale * (dw @ a.t()))
            a.grad.add_(self.scale * (b.t() @ dw))

    def grad_norm(self) -> torch.Tensor:
        return torch.sqrt(sum((p.grad.float() ** 2).sum() for p in self.A + self.B))

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
    def state_dict(self) -> dict:
        out = {}
        for t, a, b in zip(self.targets, self.A, self.B):
            out[f"base_model.model.{t.hf_module}.lora_A.weight"] = a.detach().cpu().contiguous()
            out[f"base_model.model.{t.hf_module}.lora_B.weight"] = b.detach().cpu().contiguous()
        return out

    def save(self, path: str, base_model_name: str = "") -> None:
        from safetensors.torch import save_file

        os.makedirs(path, exist_ok=True)
        save_file(self.state_dict(), os.path.join(path, "adapter_model.safetensors"), metadata={"format": "pt"})
        cfg = {"peft_type": "LORA", "r": self.rank, "lora_alpha": self.alpha, "lora_dropout": 0.0, "bias": "none",
               "target_modules": self.target_modules, "task_type": "CAUSAL_LM", "base_model_name_or_path": base_model_name}
        with open(os.path.join(path, "adapter_config.json"), "w") as f:
            json.dump(cfg, f, indent=1)
        torch.save({"optimizer": self.opt.state_dict()}, os.path.join(path, "training_state.pt"))

    def load(self, path: str, load_optimizer: bool = True) -> None:
        from safetensors.torch import load_file

        sd = load_file(os.path.join(path, "adapter_model.safetensors"))
        with torch.no_grad():
            for t, a, b in zip(self.targets, self.A, self.B):
                ka = f"base_model.model.{t.hf_module}.lora_A.weight"
                if ka in sd:
                    a.copy_(sd[ka])
                    b.copy_(sd[ka.replace("lora_A", "lora_B")])
        ts = os.path.join(path, "training_state.pt")
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
