"""Flat parameter storage shared by the trainer, the rollout engine and the weight-sync path.

All parameters of one rank live in two contiguous buffers per dtype role — ``dense`` (everything that is
replicated over expert-parallel ranks) and ``expert`` (the locally owned experts).  Every named parameter
is a view into its buffer, so the optimizer, gradient reduction and weight hand-off operate on a handful
of large flat tensors instead of thousands of small ones, and the trainer and a colocated engine can
share the very same memory (weight sync then costs a version bump, not a copy).

Native parameter names::

    embed.weight [V,H]            final_norm.weight [H]         lm_head.weight [V,H] (absent when tied)
    layers.i.ln1.weight [H]       layers.i.ln2.weight [H]
    layers.i.attn.qkv.weight [(Hq+2Hk)D, H]   (+ attn.qkv.bias)  layers.i.attn.o.weight [H, Hq*D]
    layers.i.attn.q_norm.weight [D]           layers.i.attn.k_norm.weight [D]
    layers.i.mlp.gate_up.weight [2I,H]        layers.i.mlp.down.weight [H,I]
    layers.i.moe.router.weight [E,H]          layers.i.moe.w1 [E_local,2I,H]   layers.i.moe.w2 [E_local,H,I]
    layers.i.moe.router.bias [E] (sigmoid routers)     layers.i.moe.shared.gate_up.weight [2Is,H]   ...shared.down.weight [H,Is]

The fused layouts (q|k|v rows, gate|up rows) are what the fused kernels consume; ``hf_mapping`` converts
to and from HuggingFace names, the role that megatron_to_hf/qwen3moe.py:6-117 plays in the reference.
"""
from __future__ import annotations

import hashlib
from collections import OrderedDict
from dataclasses import dataclass
from typing import Iterator, Optional

import torch

from .config import ModelConfig


@dataclass
class ParamSpec:
    name: str
    shape: tuple[int, ...]
    group: str  # "dense" | "expert"
    init: str  # "normal" | "ones" | "zeros"
    offset: int = 0

    @property
    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n


def _align(n: int, a: int = 128) -> int:
    return (n + a - 1) // a * a


def build_specs(cfg: ModelConfig, ep_size: int = 1, layers: Optional[tuple] = None, first: bool = True,
                last: bool = True) -> list[ParamSpec]:
    """All parameters of the model, or of one pipeline stage: ``layers = (lo, hi)`` keeps those decoder layers,
    ``first`` / ``last`` say whether the stage holds the embedding / the final norm and LM head (with tied embeddings
    the last stage holds a copy of the embedding as its LM head). Names always carry the global layer index."""
    assert cfg.num_experts % ep_size == 0 or not cfg.is_moe, "experts must divide evenly over EP ranks"
    H, D = cfg.hidden_size, cfg.head_dim
    lo, hi = layers if layers is not None else (0, cfg.num_layers)
    specs: list[ParamSpec] = []
    if first or (last and cfg.tie_embeddings):
        specs.append(ParamSpec("embed.weight", (cfg.vocab_size, H), "dense", "normal"))
    for i in range(lo, hi):
        p = f"layers.{i}."
        specs.append(ParamSpec(p + "ln1.weight", (H,), "dense", "ones"))
        specs.append(ParamSpec(p + "attn.qkv.weight", (cfg.qkv_dim, H), "dense", "normal"))
        if cfg.qkv_bias:
            specs.append(ParamSpec(p + "attn.qkv.bias", (cfg.qkv_dim,), "dense", "zeros"))
        if cfg.qk_norm:
            specs.append(ParamSpec(p + "attn.q_norm.weight", (D,), "dense", "ones"))
            specs.append(ParamSpec(p + "attn.k_norm.weight", (D,), "dense", "ones"))
        specs.append(ParamSpec(p + "attn.o.weight", (H, cfg.q_dim), "dense", "normal"))
        if getattr(cfg, "post_norms", False):
            specs.append(ParamSpec(p + "post_attn_ln.weight", (H,), "dense", "ones"))
            specs.append(ParamSpec(p + "post_mlp_ln.weight", (H,), "dense", "ones"))
        specs.append(ParamSpec(p + "ln2.weight", (H,), "dense", "ones"))
        if cfg.layer_is_moe(i):
            el = cfg.num_experts // ep_size
            I = cfg.moe_ffn_hidden_size
            specs.append(ParamSpec(p + "moe.router.weight", (cfg.num_experts, H), "dense", "normal"))
            if getattr(cfg, "router_bias", False):
                specs.append(ParamSpec(p + "moe.router.bias", (cfg.num_experts,), "dense", "zeros"))  # selection only: no gradient
            if getattr(cfg, "shared_expert_ffn", 0):
                Is = cfg.shared_expert_ffn
                specs.append(ParamSpec(p + "moe.shared.gate_up.weight", (2 * Is, H), "dense", "normal"))
                specs.append(ParamSpec(p + "moe.shared.down.weight", (H, Is), "dense", "normal"))
                if getattr(cfg, "shared_expert_gate", False):
                    specs.append(ParamSpec(p + "moe.shared.gate.weight", (1, H), "dense", "normal"))
            specs.append(ParamSpec(p + "moe.w1", (el, 2 * I, H), "expert", "normal"))
            specs.append(ParamSpec(p + "moe.w2", (el, H, I), "expert", "normal"))
        else:
            I = cfg.ffn_hidden_size
            specs.append(ParamSpec(p + "mlp.gate_up.weight", (2 * I, H), "dense", "normal"))
            specs.append(ParamSpec(p + "mlp.down.weight", (H, I), "dense", "normal"))
    if last:
        specs.append(ParamSpec("final_norm.weight", (H,), "dense", "ones"))
        if not cfg.tie_embeddings:
            specs.append(ParamSpec("lm_head.weight", (cfg.vocab_size, H), "dense", "normal"))
    off = {"dense": 0, "expert": 0}
    for s in specs:
        s.offset = off[s.group]
        off[s.group] += _align(s.numel)
    return specs


# ---------------------------------------------------------------------------------------------- tensor parallel
TP_SHARDED = ("attn.qkv.weight", "attn.qkv.bias", "attn.o.weight", "mlp.gate_up.weight", "mlp.down.weight")


def tp_local_config(cfg: ModelConfig, tp: int) -> ModelConfig:
    """The per-rank view of the model under tensor parallelism: heads and the dense FFN width are divided, the rest
    (hidden size, experts, vocabulary) stays. Every shape of the store and of the kernels follows from it."""
    if tp == 1:
        return cfg
    assert cfg.num_q_heads % tp == 0 and cfg.num_kv_heads % tp == 0, "tensor parallel size must divide the head counts"
    assert cfg.is_moe or cfg.ffn_hidden_size % tp == 0
    import copy

    c = copy.copy(cfg)
    c.num_q_heads, c.num_kv_heads = cfg.num_q_heads // tp, cfg.num_kv_heads // tp
    if cfg.ffn_hidden_size:
        c.ffn_hidden_size = cfg.ffn_hidden_size // tp
    return c


def is_tp_sharded(name: str) -> bool:
    return name.endswith(TP_SHARDED)


def tp_slice(cfg: ModelConfig, name: str, full: torch.Tensor, tp: int, rank: int) -> torch.Tensor:
    """Rank ``rank``'s shard of a full (global-config) tensor. qkv: the rank's q heads, k heads and v heads; o and
    down: the matching input columns; gate_up: the rank's gate rows followed by its up rows."""
    if tp == 1 or not is_tp_sharded(name):
        return full
    D = cfg.head_dim
    if name.endswith(("attn.qkv.weight", "attn.qkv.bias")):
        q, kv = cfg.q_dim, cfg.kv_dim
        ql, kl = q // tp, kv // tp
        parts = [full[rank * ql:(rank + 1) * ql], full[q + rank * kl:q + (rank + 1) * kl],
                 full[q + kv + rank * kl:q + kv + (rank + 1) * kl]]
        return torch.cat(parts, 0)
    if name.endswith("attn.o.weight"):
        ql = cfg.q_dim // tp
        return full[:, rank * ql:(rank + 1) * ql]
    if name.endswith("mlp.gate_up.weight"):
        I = cfg.ffn_hidden_size
        il = I // tp
        return torch.cat([full[rank * il:(rank + 1) * il], full[I + rank * il:I + (rank + 1) * il]], 0)
    il = cfg.ffn_hidden_size // tp  # mlp.down.weight
    return full[:, rank * il:(rank + 1) * il]


def tp_merge(cfg: ModelConfig, name: str, shards: list) -> torch.Tensor:
    """Inverse of :func:`tp_slice` for the list of all ranks' shards (rank order)."""
    tp = len(shards)
    if tp == 1 or not is_tp_sharded(name):
        return shards[0]
    if name.endswith(("attn.qkv.weight", "attn.qkv.bias")):
        ql, kl = cfg.q_dim // tp, cfg.kv_dim // tp
        return torch.cat([s[:ql] for s in shards] + [s[ql:ql + kl] for s in shards] + [s[ql + kl:] for s in shards], 0)
    if name.endswith(("attn.o.weight", "mlp.down.weight")):
        return torch.cat(shards, 1)
    il = cfg.ffn_hidden_size // tp
    return torch.cat([s[:il] for s in shards] + [s[il:] for s in shards], 0)


def _seed_for(seed: int, key: str) -> int:
    h = hashlib.blake2b(f"{seed}:{key}".encode(), digest_size=8).digest()
    return int.from_bytes(h, "little") & 0x7FFFFFFFFFFFFFFF


class ParamStore:
    """Owns the flat parameter (and optionally gradient) buffers of one rank."""

    def __init__(self, cfg: ModelConfig, device: torch.device | str = "cpu", dtype: torch.dtype = torch.bfloat16,
                 ep_size: int = 1, ep_rank: int = 0, init_std: float = 0.02, seed: int = 1234, init: bool = True,
                 meta: bool = False, tp_size: int = 1, tp_rank: int = 0, share_dense: Optional["ParamStore"] = None,
                 pp_size: int = 1, pp_rank: int = 0, pp_first_layers: Optional[int] = None,
                 pp_last_layers: Optional[int] = None, flat_override: Optional[dict] = None):
        """``flat_override``: ``{group: flat tensor}`` to use instead of allocating (e.g. views of a peer-mapped
        symmetric region that other ranks write weight updates into).
        ``cfg`` is the global model; with ``tp_size > 1`` the store holds this rank's shard (``self.cfg`` becomes
        the local view, ``self.global_cfg`` keeps the full model for conversions). With ``pp_size > 1`` it holds the
        decoder layers ``self.layer_range`` of pipeline stage ``pp_rank`` (plus embedding / head on the end stages)."""
        self.global_cfg = cfg
        self.tp_size, self.tp_rank = tp_size, tp_rank
        self.pp_size, self.pp_rank = pp_size, pp_rank
        from ..parallel.pipeline_parallel import stage_layers

        self.layer_range = stage_layers(cfg.num_layers, pp_size, pp_rank, pp_first_layers, pp_last_layers)
        self.is_first_stage, self.is_last_stage = pp_rank == 0, pp_rank == pp_size - 1
        cfg = tp_local_config(cfg, tp_size)
        self.cfg = cfg
        self.device = torch.device(device)
        self.dtype = dtype
        self.ep_size, self.ep_rank = ep_size, ep_rank
        self.specs = build_specs(cfg, ep_size, self.layer_range, self.is_first_stage, self.is_last_stage)
        self.by_name = OrderedDict((s.name, s) for s in self.specs)
        self.sizes = {g: sum(_align(s.numel) for s in self.specs if s.group == g) for g in ("dense", "expert")}
        dev = torch.device("meta") if meta else self.device
        # ``share_dense``: the replicated parameters are the other store's very buffer (a rollout replica that holds
        # all experts next to a trainer that holds its expert-parallel share)
        if share_dense is not None:
            assert share_dense.sizes["dense"] == self.sizes["dense"] and share_dense.dtype == dtype
        flat_override = flat_override or {}
        for g, t in flat_override.items():
            assert t.numel() == self.sizes[g] and t.dtype == dtype and t.is_contiguous(), f"flat_override[{g}] has the wrong size or type"
        self.flat = {g: (flat_override[g] if g in flat_override else share_dense.flat[g] if (share_dense is not None and g == "dense")
                         else torch.zeros(n, dtype=dtype, device=dev))
                     for g, n in self.sizes.items()}
        self.grad: dict[str, Optional[torch.Tensor]] = {"dense": None, "expert": None}
        self.params: "OrderedDict[str, torch.Tensor]" = OrderedDict()
        self.grads: "OrderedDict[str, torch.Tensor]" = OrderedDict()
        for s in self.specs:
            self.params[s.name] = self.flat[s.group][s.offset:s.offset + s.numel].view(s.shape)
        self.version = 0
        if init and not meta:
            self.init_weights(init_std, seed)

    # ------------------------------------------------------------------ init / access
    @torch.no_grad()
    def init_weights(self, std: float = 0.02, seed: int = 1234) -> None:
        """N(0, std) for matrices, ones for norm weights, zeros for biases. Every value is a function of
        (seed, parameter name, global expert index, element index in the unsharded tensor): any expert-, tensor- or
        pipeline-parallel factorisation builds the same model. On a CUDA device the values come from the extension's
        counter-based generator (one launch per tensor); on the CPU from seeded ``torch.Generator`` streams."""
        C = None
        if self.device.type == "cuda":
            from ..ops import _ext

            C = _ext.load(required=False)
        gen = torch.Generator(device=self.device) if C is None else None
        gshapes = {g.name: g.shape for g in build_specs(self.global_cfg, self.ep_size)} if self.tp_size > 1 else {}
        el = self.cfg.num_experts // self.ep_size if self.cfg.is_moe else 0

        def draw(dst: torch.Tensor, key: str) -> None:
            """Fill the contiguous view ``dst`` (a whole logical tensor) with N(0, std) under ``key``."""
            k = _seed_for(seed, key)
            if C is not None:
                C.init_normal(dst, k, std)
                return
            gen.manual_seed(k)
            flat = dst.view(-1)
            chunk = 1 << 26
            for a in range(0, flat.numel(), chunk):
                b = min(a + chunk, flat.numel())
                flat[a:b].copy_(torch.empty(b - a, dtype=torch.float32, device=self.device).normal_(0.0, std, generator=gen))

        for s in self.specs:
            p = self.params[s.name]
            if s.init == "ones":
                p.fill_(1.0)
            elif s.init == "zeros":
                p.zero_()
            elif s.group == "expert":
                # one stream per *global* expert so that any EP factorisation builds the same model
                for le in range(el):
                    draw(p[le], f"{s.name}:{self.ep_rank * el + le}")
            elif self.tp_size > 1 and is_tp_sharded(s.name):
                # draw the full tensor of the global model and keep this rank's shard
                full = torch.empty(gshapes[s.name], dtype=torch.float32, device=self.device)
                draw(full, s.name)
                p.copy_(tp_slice(self.global_cfg, s.name, full, self.tp_size, self.tp_rank))
                del full
            else:
                draw(p, s.name)

    def __getitem__(self, name: str) -> torch.Tensor:
        return self.params[name]

    def named_parameters(self) -> Iterator[tuple[str, torch.Tensor]]:
        return iter(self.params.items())

    def lm_head(self) -> torch.Tensor:
        return self.params["embed.weight"] if self.cfg.tie_embeddings else self.params["lm_head.weight"]

    # ------------------------------------------------------------------ gradients
    def allocate_grads(self, dtype: torch.dtype = torch.float32, expert_dtype: Optional[torch.dtype] = None,
                       expert_storage: Optional[torch.Tensor] = None) -> None:
        """Flat gradient buffers per group. ``expert_storage`` (uint8) places the expert gradients in memory
        the caller owns — the colocated loop lends the same bytes to the KV cache between training steps."""
        for g, n in self.sizes.items():
            dt = expert_dtype if (g == "expert" and expert_dtype is not None) else dtype
            pinned = getattr(self, "_pinned_grads", {}).get(g)
            if pinned is not None:
                self.grad[g] = pinned
                continue
            if g == "expert" and expert_storage is not None and n > 0:
                nbytes = n * torch.empty((), dtype=dt).element_size()
                assert expert_storage.dtype == torch.uint8 and expert_storage.numel() >= nbytes
                self.grad[g] = None
                self.grad[g] = expert_storage[:nbytes].view(dt)
                self.grad[g].zero_()
            elif self.grad[g] is None or self.grad[g].dtype != dt:
                self.grad[g] = None
                self.grad[g] = torch.zeros(n, dtype=dt, device=self.device)
        self.grads.clear()
        for s in self.specs:
            self.grads[s.name] = self.grad[s.group][s.offset:s.offset + s.numel].view(s.shape)

    def rebind_flat(self, group: str, tensor: torch.Tensor) -> None:
        """Move a flat parameter buffer to caller-provided storage (same size and dtype, contents already copied):
        every named parameter of the group becomes a view of the new buffer."""
        assert tensor.numel() == self.flat[group].numel() and tensor.dtype == self.flat[group].dtype
        self.flat[group] = tensor
        for s in self.specs:
            if s.group == group:
                self.params[s.name] = tensor[s.offset:s.offset + s.numel].view(s.shape)

    def pin_grad_storage(self, group: str, tensor: torch.Tensor) -> None:
        """Keep the group's gradients in caller-provided storage from now on (survives free / allocate cycles)."""
        assert tensor.numel() == self.sizes[group]
        if not hasattr(self, "_pinned_grads"):
            self._pinned_grads = {}
        self._pinned_grads[group] = tensor
        had = bool(self.grads)
        self.grad[group] = tensor
        if had:
            for s in self.specs:
                if s.group == group:
                    self.grads[s.name] = tensor[s.offset:s.offset + s.numel].view(s.shape)

    def zero_grads(self) -> None:
        for g in self.grad.values():
            if g is not None:
                g.zero_()

    def free_grads(self) -> None:
        self.grad = {"dense": None, "expert": None}
        self.grads.clear()

    def num_local_params(self) -> int:
        return sum(s.numel for s in self.specs)

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.flat.values())

    @torch.no_grad()
    def copy_from(self, other: "ParamStore") -> None:
        for g in self.flat:
            self.flat[g].copy_(other.flat[g].to(self.flat[g].dtype))
        self.version = other.version

    def checksum(self) -> dict[str, float]:
        """Cheap per-group checksum used by the weight-update equality checks."""
        return {g: float(t.float().abs().sum().item()) if t.numel() else 0.0 for g, t in self.flat.items()}
