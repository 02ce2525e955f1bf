"""Pure-PyTorch execution of the Qwen3 dense / MoE decoder over a ``ParamStore``.

This is (a) the autograd oracle the hand-written sm_100a forward/backward is tested against, and (b) the
compute path of the CPU/gloo configuration (tiny fp32 model, world size 2), for both the trainer and
the rollout engine.  Layout conventions are shared with ``b200_impl``: packed tokens ``[T]`` with
``cu_seqlens``, fused qkv / gate_up weights, rotate-half RoPE, softmax->top-k->renormalise routing.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch
import torch.nn.functional as F

from ..ops import reference as R
from .config import ModelConfig
from .params import ParamStore


@dataclass
class InferMeta:
    """Attention metadata of one engine forward.

    prefill: ``cu_seqlens`` over the packed new tokens, ``slot_mapping[t]`` = cache slot of token t.
    decode : one token per sequence, ``block_table`` [B, max_pages], ``seq_lens`` [B] (including the new token).
    """
    is_prefill: bool
    cu_seqlens: Optional[torch.Tensor] = None
    max_seqlen: int = 0
    slot_mapping: Optional[torch.Tensor] = None
    block_table: Optional[torch.Tensor] = None
    seq_lens: Optional[torch.Tensor] = None
    page_size: int = 16
    cu_list: list = field(default_factory=list)
    prefix: Optional["PrefixInfo"] = None  # prefill only: part of every sequence is already in the KV cache


@dataclass
class PrefixInfo:
    """Prefill over sequences whose first ``prefix_lens[i]`` tokens are cached: the pass computes only the remaining
    ``new_lens[i]`` tokens, and the attention reads keys / values of the cached part from the cache slots ``pre_slots``.
    ``pre_dst`` / ``new_dst`` place both parts in one packed key / value tensor per layer (sequence i: its cached rows,
    then its new rows), which is what the attention kernel's tile table (``tiles``) indexes."""
    prefix_lens: list
    new_lens: list
    pre_slots: torch.Tensor
    pre_dst: torch.Tensor
    new_dst: torch.Tensor
    total: int
    tiles: Optional[torch.Tensor] = None

    @classmethod
    def build(cls, prefix_lens, new_lens, pre_slots: torch.Tensor, device) -> "PrefixInfo":
        pre_dst, new_dst, start = [], [], 0
        for c, n in zip(prefix_lens, new_lens):
            pre_dst.append(torch.arange(start, start + c))
            new_dst.append(torch.arange(start + c, start + c + n))
            start += c + n
        from ..ops.attention import build_tiles

        return cls(list(prefix_lens), list(new_lens), pre_slots.to(device=device, dtype=torch.int64),
                   torch.cat(pre_dst).to(device), torch.cat(new_dst).to(device), start,
                   build_tiles(new_lens, prefix_lens).to(device))

    def full_kv(self, k_new: torch.Tensor, v_new: torch.Tensor, kc: torch.Tensor, vc: torch.Tensor):
        """Packed keys / values of every sequence: cached rows gathered from the cache, then the rows of this pass."""
        kf = k_new.new_empty((self.total,) + tuple(k_new.shape[1:]))
        vf = v_new.new_empty((self.total,) + tuple(v_new.shape[1:]))
        kf[self.new_dst], vf[self.new_dst] = k_new, v_new
        kf[self.pre_dst] = kc[self.pre_slots].to(k_new.dtype)
        vf[self.pre_dst] = vc[self.pre_slots].to(v_new.dtype)
        return kf, vf


class TorchQwen3:
    def __init__(self, cfg: ModelConfig, store: ParamStore, ep_group=None):
        self.cfg = cfg
        self.store = store
        self.ep_group = ep_group
        self.cp_ctx = None  # (sample lengths, cp size, cp rank, group) while a context-parallel micro-batch is processed
        if store.ep_size != 1:
            raise NotImplementedError("the PyTorch execution path keeps all experts on every rank")

    # ------------------------------------------------------------------ blocks
    def _attn_block(self, i, x, positions, cu, meta: Optional[InferMeta], kv_cache):
        cfg, P = self.cfg, self.store.params
        p = f"layers.{i}."
        h = R.rmsnorm(x, P[p + "ln1.weight"], cfg.rms_eps)
        qkv = F.linear(h, P[p + "attn.qkv.weight"], P.get(p + "attn.qkv.bias"))
        inv_freq = None
        rdim = getattr(cfg, "rotary_dim", 0)
        if cfg.rope_scaling:
            if getattr(self, "_inv_freq", None) is None or self._inv_freq.device != qkv.device:
                self._inv_freq = R.rope_inv_freq(rdim or cfg.head_dim, cfg.rope_theta, cfg.rope_scaling, qkv.device)
            inv_freq = self._inv_freq
        q, k, v = R.qk_norm_rope(qkv, P.get(p + "attn.q_norm.weight"), P.get(p + "attn.k_norm.weight"), positions,
                                 cfg.num_q_heads, cfg.num_kv_heads, cfg.head_dim, cfg.rope_theta, cfg.rms_eps, inv_freq, rdim)
        scale = cfg.head_dim ** -0.5
        if meta is None or meta.is_prefill:
            if kv_cache is not None:
                kc, vc = kv_cache[i]
                kc[meta.slot_mapping.long()] = k.to(kc.dtype)
                vc[meta.slot_mapping.long()] = v.to(vc.dtype)
            if self.cp_ctx is not None and meta is None:
                from ..parallel.context_parallel import attention_zigzag, gather_kv_autograd

                lens, cp, rank, group = self.cp_ctx[:4]
                layout = self.cp_ctx[5] if len(self.cp_ctx) > 5 else "zigzag"
                if len(self.cp_ctx) > 4 and self.cp_ctx[4] == "a2a":
                    # Ulysses: trade the sequence shard for a head shard, attend over whole sequences, trade back
                    from ..parallel.context_parallel import heads_to_sequence, sequence_to_heads

                    qf, kf, vf = (heads_to_sequence(t, lens, cp, rank, group, layout) for t in (q, k, v))
                    full_cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0).tolist()), dtype=torch.int32, device=q.device)
                    att = sequence_to_heads(R.attention_varlen(qf, kf, vf, full_cu, scale), lens, cp, rank, group, layout)
                else:
                    kf, vf = gather_kv_autograd(k, v, lens, cp, rank, group, layout)
                    att = attention_zigzag(q, kf, vf, lens, cp, rank, scale, layout)
            elif meta is not None and meta.prefix is not None:
                # prefill behind a cached prefix: every sequence's new queries attend to its cached + new keys
                pf = meta.prefix
                kf, vf = pf.full_kv(k, v, *kv_cache[i])
                outs, q0, s0 = [], 0, 0
                for c, n in zip(pf.prefix_lens, pf.new_lens):
                    outs.append(R.attention_prefix(q[q0:q0 + n], kf[s0:s0 + c + n], vf[s0:s0 + c + n], c, scale))
                    q0, s0 = q0 + n, s0 + c + n
                att = torch.cat(outs, 0)
            else:
                att = R.attention_varlen(q, k, v, cu, scale)
        else:
            kc, vc = kv_cache[i]
            kc[meta.slot_mapping.long()] = k.to(kc.dtype)
            vc[meta.slot_mapping.long()] = v.to(vc.dtype)
            outs = []
            ps = meta.page_size
            for b in range(q.shape[0]):
                L = int(meta.seq_lens[b])
                pages = meta.block_table[b, : (L + ps - 1) // ps].long()
                slots = (pages[:, None] * ps + torch.arange(ps, device=q.device)[None, :]).reshape(-1)[:L]
                outs.append(R.attention_prefix(q[b:b + 1], kc[slots].to(q.dtype), vc[slots].to(q.dtype), L - 1, scale))
            att = torch.cat(outs, 0)
        o = F.linear(att.reshape(att.shape[0], -1), P[p + "attn.o.weight"])
        if getattr(cfg, "post_norms", False):
            o = R.rmsnorm(o, P[p + "post_attn_ln.weight"], cfg.rms_eps)
        return x + o

    def _mlp_block(self, i, x, replay_ids=None, record=None):
        cfg, P = self.cfg, self.store.params
        p = f"layers.{i}."
        h = R.rmsnorm(x, P[p + "ln2.weight"], cfg.rms_eps)
        if cfg.layer_is_moe(i):
            logits = F.linear(h.float(), P[p + "moe.router.weight"].float())
            if getattr(cfg, "router_score", "softmax") == "sigmoid":
                ids, w, _ = R.router_sigmoid_topk(logits, cfg.moe_top_k, cfg.norm_topk_prob, P.get(p + "moe.router.bias"),
                                                  cfg.routed_scaling_factor, cfg.n_group, cfg.topk_group, replay_ids)
            else:
                ids, w, _ = R.router_topk(logits, cfg.moe_top_k, cfg.norm_topk_prob, replay_ids)
            if record is not None:
                record.append(ids)
            y = R.moe_experts(h, ids, w.to(h.dtype) if h.dtype != torch.float32 else w, P[p + "moe.w1"], P[p + "moe.w2"])
            if getattr(cfg, "shared_expert_ffn", 0):
                sh = F.linear(R.swiglu(F.linear(h, P[p + "moe.shared.gate_up.weight"])), P[p + "moe.shared.down.weight"])
                if getattr(cfg, "shared_expert_gate", False):
                    sh = torch.sigmoid(F.linear(h, P[p + "moe.shared.gate.weight"])) * sh
                y = y + sh
        else:
            y = F.linear(R.swiglu(F.linear(h, P[p + "mlp.gate_up.weight"])), P[p + "mlp.down.weight"])
        if getattr(cfg, "post_norms", False):
            y = R.rmsnorm(y, P[p + "post_mlp_ln.weight"], cfg.rms_eps)
        return x + y

    # ------------------------------------------------------------------ forward
    def forward_hidden(self, tokens, positions, cu_seqlens, meta: Optional[InferMeta] = None, kv_cache=None,
                       replay: Optional[torch.Tensor] = None, record: Optional[list] = None,
                       x_in: Optional[torch.Tensor] = None):
        """tokens/positions [T] -> final-normed hidden [T,H]. ``replay`` is int32 [T, n_moe_layers, K]. Under
        pipeline parallelism this runs the stage's layers: later stages start from ``x_in``, every stage but the last
        returns the raw hidden states for the next one."""
        cfg, P = self.cfg, self.store.params
        begin = getattr(self.store, "begin_pass", None)
        if begin is not None:
            begin()
        lo, hi = getattr(self.store, "layer_range", (0, cfg.num_layers))
        x = F.embedding(tokens.long(), P["embed.weight"]) if getattr(self.store, "is_first_stage", True) else x_in
        moe_idx = sum(cfg.layer_is_moe(j) for j in range(lo))
        for i in range(lo, hi):
            x = self._attn_block(i, x, positions, cu_seqlens, meta, kv_cache)
            rid = None
            if cfg.layer_is_moe(i):
                if replay is not None:
                    rid = replay[:, moe_idx]
                moe_idx += 1
            x = self._mlp_block(i, x, rid, record)
        if not getattr(self.store, "is_last_stage", True):
            return x
        return R.rmsnorm(x, P["final_norm.weight"], cfg.rms_eps)

    def logits(self, hidden_rows):
        return F.linear(hidden_rows, self.store.lm_head())

    def logprobs_entropy(self, hidden_rows, targets, inv_temp: float, chunk: int = 4096):
        lps, ents = [], []
        for a in range(0, hidden_rows.shape[0], chunk):
            lp, ent = R.logprob_entropy(self.logits(hidden_rows[a:a + chunk]), targets[a:a + chunk], inv_temp)
            lps.append(lp)
            ents.append(ent)
        if not lps:
            z = hidden_rows.new_zeros((0,), dtype=torch.float32)
            return z, z.clone()
        return torch.cat(lps), torch.cat(ents)

    # ------------------------------------------------------------------ trainer API (autograd)
    def forward_logprobs(self, tokens, positions, cu_seqlens, row_index, targets, inv_temp, replay=None, record=None,
                         with_grad: bool = False, x_in: Optional[torch.Tensor] = None, max_seqlen: int = 0):
        """Log-probs/entropy of ``targets`` predicted at packed rows ``row_index``."""
        ctx = torch.enable_grad() if with_grad else torch.no_grad()
        with ctx:
            hidden = self.forward_hidden(tokens, positions, cu_seqlens, replay=replay, record=record, x_in=x_in)
            return self.logprobs_entropy(hidden[row_index.long()], targets, inv_temp)

    def set_requires_grad(self, flag: bool) -> None:
        hook = getattr(self.store, "on_requires_grad", None)
        if hook is not None:
            hook(flag)  # a sharded store: the leaves are its shard buffers, full parameters are gathered under autograd
            return
        for t in self.store.flat.values():
            t.requires_grad_(flag)
        # views were created before requires_grad was set; rebuild them so autograd tracks them
        for s in self.store.specs:
            self.store.params[s.name] = self.store.flat[s.group][s.offset:s.offset + s.numel].view(s.shape)

    def accumulate_autograd_grads(self) -> None:
        """Move ``flat.grad`` produced by autograd into the persistent gradient buffers."""
        for g, t in self.store.flat.items():
            if t.grad is not None and self.store.grad[g] is not None:
                self.store.grad[g].add_(t.grad.to(self.store.grad[g].dtype))
                t.grad = None
