"""Native parameter layout <-> HuggingFace names (Qwen3 / Qwen3-MoE / Qwen2 / Llama / Mistral / Mixtral conventions).

``to_hf`` splits the fused tensors (q|k|v rows, gate|up rows, stacked experts) into the per-projection
tensors an HF checkpoint or an external engine expects; ``from_hf`` is the inverse.  This is the role of
the per-architecture converters in the reference's
miles/backends/megatron_utils/megatron_to_hf/{qwen2,qwen3moe}.py (there the source layout is
Megatron's interleaved per-group QKV; here the fused layout is plain row concatenation, so the
conversion is pure slicing without reshuffles).
"""
from __future__ import annotations

import re
from typing import Iterator

import torch

from .config import ModelConfig


def to_hf(cfg: ModelConfig, name: str, t: torch.Tensor, expert_offset: int = 0) -> list:
    """One native tensor -> list of (hf_name, tensor view)."""
    if name == "embed.weight":
        return [("model.embed_tokens.weight", t)]
    if name == "final_norm.weight":
        return [("model.norm.weight", t)]
    if name == "lm_head.weight":
        return [("lm_head.weight", t)]
    m = re.match(r"layers\.(\d+)\.(.+)", name)
    assert m, f"unknown parameter {name}"
    i, rest = int(m.group(1)), m.group(2)
    p = f"model.layers.{i}."
    q, kv = cfg.q_dim, cfg.kv_dim
    if rest == "ln1.weight":
        return [(p + "input_layernorm.weight", t)]
    if rest == "ln2.weight":
        return [(p + "post_attention_layernorm.weight", t)]
    if rest == "post_attn_ln.weight":
        return [(p + "post_self_attn_layernorm.weight", t)]
    if rest == "post_mlp_ln.weight":
        return [(p + "post_mlp_layernorm.weight", t)]
    fused_names = getattr(cfg, "family", "") == "phi3"  # one qkv_proj and one gate_up_proj tensor, in this package's row order
    if rest in ("attn.qkv.weight", "attn.qkv.bias") and fused_names:
        return [(p + f"self_attn.qkv_proj.{rest.rsplit('.', 1)[1]}", t)]
    if rest == "mlp.gate_up.weight" and fused_names:
        return [(p + "mlp.gate_up_proj.weight", t)]
    if rest in ("attn.qkv.weight", "attn.qkv.bias"):
        sfx = rest.rsplit(".", 1)[1]
        return [(p + f"self_attn.q_proj.{sfx}", t[:q]), (p + f"self_attn.k_proj.{sfx}", t[q:q + kv]),
                (p + f"self_attn.v_proj.{sfx}", t[q + kv:])]
    if rest == "attn.q_norm.weight":
        return [(p + "self_attn.q_norm.weight", t)]
    if rest == "attn.k_norm.weight":
        return [(p + "self_attn.k_norm.weight", t)]
    if rest == "attn.o.weight":
        return [(p + "self_attn.o_proj.weight", t)]
    if rest == "mlp.gate_up.weight" and getattr(cfg, "family", "") == "glm4":
        return [(p + "mlp.gate_up_proj.weight", t)]  # fused in the checkpoint too: gate rows, then up rows
    if rest == "mlp.gate_up.weight":
        I = t.shape[0] // 2
        return [(p + "mlp.gate_proj.weight", t[:I]), (p + "mlp.up_proj.weight", t[I:])]
    if rest == "mlp.down.weight":
        return [(p + "mlp.down_proj.weight", t)]
    if rest == "moe.router.bias":
        return [(p + "mlp.gate.e_score_correction_bias", t)]
    shared = "mlp.shared_expert." if getattr(cfg, "family", "") == "qwen2_moe" else "mlp.shared_experts."
    if rest == "moe.shared.gate_up.weight":
        I = t.shape[0] // 2
        return [(p + shared + "gate_proj.weight", t[:I]), (p + shared + "up_proj.weight", t[I:])]
    if rest == "moe.shared.down.weight":
        return [(p + shared + "down_proj.weight", t)]
    if rest == "moe.shared.gate.weight":
        return [(p + "mlp.shared_expert_gate.weight", t)]
    mixtral = getattr(cfg, "family", "") == "mixtral"  # block_sparse_moe.{gate, experts.N.w1 (gate) / w3 (up) / w2 (down)}
    if rest == "moe.router.weight":
        return [(p + ("block_sparse_moe.gate.weight" if mixtral else "mlp.gate.weight"), t)]
    if rest == "moe.w1":
        I = t.shape[1] // 2
        out = []
        for e in range(t.shape[0]):
            ge = expert_offset + e
            if mixtral:
                out += [(p + f"block_sparse_moe.experts.{ge}.w1.weight", t[e, :I]), (p + f"block_sparse_moe.experts.{ge}.w3.weight", t[e, I:])]
            else:
                out += [(p + f"mlp.experts.{ge}.gate_proj.weight", t[e, :I]), (p + f"mlp.experts.{ge}.up_proj.weight", t[e, I:])]
        return out
    if rest == "moe.w2":
        if mixtral:
            return [(p + f"block_sparse_moe.experts.{expert_offset + e}.w2.weight", t[e]) for e in range(t.shape[0])]
        return [(p + f"mlp.experts.{expert_offset + e}.down_proj.weight", t[e]) for e in range(t.shape[0])]
    raise KeyError(name)


def _rope_rows(cfg: ModelConfig, t: torch.Tensor, heads: int, to_checkpoint: bool) -> torch.Tensor:
    """Reorder the rotary rows of a query / key projection (weight ``[heads * D, H]`` or bias ``[heads * D]``) between the
    checkpoint's interleaved pairing (2i with 2i + 1) and the model's halves (i with i + R / 2). Returns a new tensor."""
    D, R = cfg.head_dim, (cfg.rotary_dim or cfg.head_dim)
    x = t.reshape(heads, D, *t.shape[1:]).clone()
    rot = x[:, :R]
    if to_checkpoint:
        out = torch.empty_like(rot)
        out[:, 0::2], out[:, 1::2] = rot[:, :R // 2], rot[:, R // 2:]
    else:
        out = torch.cat([rot[:, 0::2], rot[:, 1::2]], dim=1)
    x[:, :R] = out
    return x.reshape(t.shape)


def _rope_heads(cfg: ModelConfig, hf_name: str) -> int:
    """How many heads a HuggingFace tensor's rotary rows cover, 0 for tensors without any (models whose checkpoints pair
    rotary dimensions like the model does need nothing)."""
    if not getattr(cfg, "rope_interleaved", False):
        return 0
    if ".self_attn.q_proj." in hf_name:
        return cfg.num_q_heads
    if ".self_attn.k_proj." in hf_name:
        return cfg.num_kv_heads
    return 0


def hf_names(cfg: ModelConfig, store, tp_group=None) -> Iterator[tuple]:
    """Iterate (hf_name, tensor) over every local parameter of ``store``. Under tensor parallelism the sharded
    tensors are gathered over ``tp_group`` first (a collective: every rank of the group must iterate), which is
    the all-gather the reference performs per parameter (update_weight/common.py:189-221)."""
    from .params import is_tp_sharded, tp_merge

    gcfg = getattr(store, "global_cfg", cfg)
    tp = getattr(store, "tp_size", 1)
    el = cfg.num_experts // store.ep_size if cfg.is_moe else 0
    for name, t in store.named_parameters():
        if tp > 1 and is_tp_sharded(name):
            import torch.distributed as dist

            parts = [torch.empty_like(t) for _ in range(tp)]
            dist.all_gather(parts, t.contiguous(), group=tp_group)
            t = tp_merge(gcfg, name, parts)
        for hf_name, view in to_hf(gcfg, name, t, expert_offset=store.ep_rank * el):
            heads = _rope_heads(gcfg, hf_name)
            yield (hf_name, _rope_rows(gcfg, view, heads, to_checkpoint=True) if heads else view)


def param_or_hf_view(cfg: ModelConfig, store, name: str) -> torch.Tensor:
    """The destination of a weight that arrives under ``name``: a native parameter name, or a HuggingFace tensor name,
    which maps to a view of the (possibly fused) native parameter. Because HF pieces land in views (q / k / v rows of
    the fused QKV, gate / up rows of the fused first MLP matrix, one expert's rows of the stacked expert tensors), a
    sender may deliver them in any order and split them over buckets as it likes: no group of tensors has to arrive in
    one call (the reference needs such atomic groups for loaders that fuse on arrival,
    miles/backends/megatron_utils/update_weight/common.py:21-131)."""
    if name in store.params:
        return store.params[name]
    if _rope_heads(getattr(store, "global_cfg", cfg), name):
        raise NotImplementedError(f"{name}: this model's checkpoints interleave rotary rows; send the fused native parameter "
                                  "(attn.qkv.weight) instead of the HuggingFace piece")
    views = getattr(store, "_hf_views", None)
    if views is None:
        assert getattr(store, "tp_size", 1) == 1, "HF-named updates address unsharded parameters"
        el = cfg.num_experts // store.ep_size if cfg.is_moe else 0
        views = {}
        for pname, dst in store.named_parameters():
            for hf_name, view in to_hf(getattr(store, "global_cfg", cfg), pname, dst, expert_offset=store.ep_rank * el):
                views[hf_name] = view
        store._hf_views = views
    if name not in views:
        raise KeyError(f"{name} is neither a parameter of this model nor one of its HuggingFace tensor names")
    return views[name]


def from_hf(cfg: ModelConfig, store, get_tensor, strict: bool = True) -> int:
    """Fill ``store`` from HF tensors; ``get_tensor(hf_name) -> tensor | None``. Returns #tensors loaded."""
    from .params import build_specs, is_tp_sharded, tp_slice

    gcfg = getattr(store, "global_cfg", cfg)
    tp = getattr(store, "tp_size", 1)
    gshapes = {s.name: s.shape for s in build_specs(gcfg, store.ep_size)} if tp > 1 else {}
    el = cfg.num_experts // store.ep_size if cfg.is_moe else 0
    n = 0
    with torch.no_grad():
        for name, dst in store.named_parameters():
            if tp > 1 and is_tp_sharded(name):
                # assemble the full tensor of the global model on the host, keep this rank's shard
                full = torch.empty(gshapes[name], dtype=dst.dtype)
                for hf_name, view in to_hf(gcfg, name, full):
                    src = get_tensor(hf_name)
                    if src is None:
                        if strict:
                            raise KeyError(f"missing tensor {hf_name} in checkpoint")
                        continue
                    heads = _rope_heads(gcfg, hf_name)
                    view.copy_((_rope_rows(gcfg, src, heads, to_checkpoint=False) if heads else src).to(view.dtype))
                    n += 1
                dst.copy_(tp_slice(gcfg, name, full, tp, store.tp_rank))
                continue
            for hf_name, view in to_hf(gcfg, name, dst, expert_offset=store.ep_rank * el):
                src = get_tensor(hf_name)
                if src is None:
                    if name == "lm_head.weight":
                        src = get_tensor("model.embed_tokens.weight")
                    if src is None:
                        if strict:
                            raise KeyError(f"missing tensor {hf_name} in checkpoint")
                        continue
                heads = _rope_heads(gcfg, hf_name)
                view.copy_((_rope_rows(gcfg, src, heads, to_checkpoint=False) if heads else src).to(view.dtype))
                n += 1
    return n
