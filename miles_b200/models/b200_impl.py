"""Hand-scheduled sm_100a execution of the Qwen3 dense / MoE decoder (training and inference).

There is no autograd graph and no tracing compiler on this path: forward and backward of a decoder
layer are explicit sequences of kernel launches (tcgen05 GEMMs, fused norm / rope / swiglu / routing
kernels), activations are recomputed layer by layer in the backward pass (only each layer's input is
kept, the "full recompute" policy of the reference recipe scripts/run_qwen3_30b_a3b.py:168-175), and
weight gradients are accumulated by the GEMM epilogue directly into the persistent flat gradient buffer
(the role of Megatron's ``main_grad`` + gradient-accumulation fusion).

The same object serves the rollout engine (prefill and paged-KV decode), so trainer and engine share
kernels and reduction orders — the basis for trainer/rollout log-prob parity.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..ops import _ext
from ..ops.attention import TileCache
from .config import ModelConfig
from .params import ParamStore
from .torch_impl import InferMeta


@dataclass
class MoeCtx:
    ids: torch.Tensor
    w: torch.Tensor
    probs: torch.Tensor
    offsets: torch.Tensor
    dest: torch.Tensor
    src: torch.Tensor
    tile_group: torch.Tensor
    num_tiles: torch.Tensor
    max_rows: int
    align: int = 1


class B200Qwen3:
    def __init__(self, cfg: ModelConfig, store: ParamStore, ep=None, tp=None):
        assert cfg.head_dim == 128, "the sm_100a attention/rope kernels are specialised for head_dim 128"
        self.cfg = store.cfg  # under tensor parallelism: this rank's view (local head counts, local FFN width)
        self.store = store
        self.ep = ep  # expert-parallel dispatcher (None = all experts local)
        self.tp = tp if (tp is not None and tp.n > 1) else None  # tensor-parallel exchange (None = not sharded)
        assert not (self.tp is not None and ep is not None), "tensor parallel attention with expert parallel MoE is not supported"
        self.C = _ext.load(required=True)
        self.dev = store.device
        self.status = torch.zeros(1, dtype=torch.int32, device=self.dev)
        self.launches = 0  # number of this library's kernels launched (reported by the benchmark)
        self._decode_scratch: Optional[torch.Tensor] = None
        self._tiles = TileCache()
        self.cp_ctx = None  # (sample lengths, cp size, cp rank, group, comm, layout) while a context-parallel micro-batch runs
        self._ident: Optional[torch.Tensor] = None
        self.small_decode = True  # weight-streaming kernels for decode steps of at most SMALL_T rows
        self.lm_chunk = 2048      # rows of the LM head per pass (--log-probs-chunk-size)

    def attention(self, q, k, v, cu):
        """Causal attention over packed sequences: returns (out [T, Hq, 128], lse [Hq, T]).

        Under context parallelism (``cp_ctx`` set by the trainer: the rows are this rank's shard of every sequence)
        the sequence shard is traded for a head shard with one all-to-all per tensor, the kernel attends over whole
        sequences with ``Hq / cp`` query heads, and the output is traded back; what the backward needs in that layout
        travels in the second return value. NVSwitch gives the all-to-all full bandwidth between every pair, so this
        layout, not a ring of K/V blocks, is the one built for this path."""
        if self.cp_ctx is not None:
            return self._attention_cp(q, k, v)
        out, lse = self.C.flash_attn_fwd(q, k, v, self._tiles.get(cu), self.cfg.head_dim ** -0.5, self.status)
        self.launches += 1
        return out, lse

    def attention_backward(self, q, k, v, out, d_out, lse, cu):
        """dQ, dK, dV of :meth:`attention` from its output and log-sum-exp (tcgen05 kernel, csrc/attention_bwd.cu)."""
        if isinstance(lse, tuple):
            return self._attention_cp_backward(d_out, lse)
        dq, dk, dv = self.C.flash_attn_bwd(q, k, v, out, d_out.contiguous(), lse, self._tiles.get_bwd(cu),
                                           self.cfg.head_dim ** -0.5, self.status)
        self.launches += 3
        return dq, dk, dv

    def _cp_full_cu(self, lens):
        key = tuple(lens)
        if getattr(self, "_cp_cu_key", None) != key:
            self._cp_cu = torch.tensor([0] + list(torch.tensor(list(lens)).cumsum(0).tolist()), dtype=torch.int32, device=self.dev)
            self._cp_cu_key = key
        return self._cp_cu

    def _attention_cp(self, q, k, v):
        from ..parallel.context_parallel import heads_to_sequence, sequence_to_heads

        lens, cp, rank, group = self.cp_ctx[:4]
        layout = self.cp_ctx[5] if len(self.cp_ctx) > 5 else "zigzag"
        cfg = self.cfg
        assert cfg.num_kv_heads % cp == 0, (f"context parallelism on this path shards the {cfg.num_kv_heads} key / value heads "
                                            f"over the {cp} ranks (all-to-all layout)")
        qf, kf, vf = (heads_to_sequence(t.contiguous(), lens, cp, rank, group, layout).contiguous() for t in (q, k, v))
        cu = self._cp_full_cu(lens)
        out_f, lse_f = self.C.flash_attn_fwd(qf, kf, vf, self._tiles.get(cu), cfg.head_dim ** -0.5, self.status)
        self.launches += 1
        out = sequence_to_heads(out_f, lens, cp, rank, group, layout).contiguous()  # (a view when a rank holds one head)
        return out, (lse_f, qf, kf, vf, out_f, cu)

    def _attention_cp_backward(self, d_out, saved):
        from ..parallel.context_parallel import heads_to_sequence, sequence_to_heads

        lens, cp, rank, group = self.cp_ctx[:4]
        layout = self.cp_ctx[5] if len(self.cp_ctx) > 5 else "zigzag"
        lse_f, qf, kf, vf, out_f, cu = saved
        do_f = heads_to_sequence(d_out.contiguous(), lens, cp, rank, group, layout).contiguous()
        dqf, dkf, dvf = self.C.flash_attn_bwd(qf, kf, vf, out_f, do_f, lse_f, self._tiles.get_bwd(cu), self.cfg.head_dim ** -0.5,
                                              self.status)
        self.launches += 3
        return tuple(sequence_to_heads(t, lens, cp, rank, group, layout).contiguous() for t in (dqf, dkf, dvf))

    # ------------------------------------------------------------------ GEMM helpers
    def _gemm(self, a, b, out, a_mn=False, b_mn=False, acc=False):
        self.C.gemm(a, b, out, a_mn, b_mn, acc, 0, self.status)
        self.launches += 1
        return out

    # ------------------------------------------------------------------ block-scaled inference weights
    MX_SUFFIXES = ("attn.qkv.weight", "attn.o.weight", "mlp.gate_up.weight", "mlp.down.weight", "moe.w1", "moe.w2")

    def enable_block_scaled(self, kind: str) -> int:
        """Serve the projections and experts from MXFP8 / NVFP4 copies of the weights (`csrc/gemm_mx.cu`) whenever
        more than 32 rows are multiplied; the few-row decode kernels keep streaming the bf16 weights. Meant for a
        model object that only the rollout engine uses. Call again (or `refresh_block_scaled`) after a weight update.
        Returns the number of tensors quantised."""
        from ..ops.mx_gemm import quantize_operand

        step = 128 if kind == "mxfp8" else 256
        self.mx_kind, self.mx = kind, {}
        for name, w in self.store.params.items():
            if not name.endswith(self.MX_SUFFIXES):
                continue
            w2 = w.reshape(-1, w.shape[-1])
            if w2.shape[1] % step or w2.shape[0] % 128:
                continue
            self.mx[w.data_ptr()] = quantize_operand(w2, kind)
        return len(self.mx)

    def use_block_scaled(self, kind: str, operands: dict) -> None:
        """Serve from block-scaled copies that something else keeps up to date (``{parameter name: MxOperand}``, e.g.
        the buffers a peer-memory weight push quantises into)."""
        self.mx_kind, self.mx_external = kind, True
        self.mx = {self.store.params[n].data_ptr(): op for n, op in operands.items() if n in self.store.params}

    def refresh_block_scaled(self) -> None:
        if getattr(self, "mx_external", False):
            return
        if getattr(self, "mx", None):
            self.enable_block_scaled(self.mx_kind)

    def _mx_linear(self, x, wq, tile_group=None, num_tiles=None, n: int = 0, amax=None):
        from ..ops.mx_gemm import mx_linear, quantize_operand

        xq = quantize_operand(x, self.mx_kind, amax)
        self.launches += 3
        return mx_linear(xq, wq, self.status, tile_group, num_tiles, n)

    def linear(self, x, w, out_dtype=torch.bfloat16):
        T, (N, K) = x.shape[0], w.shape
        mx = getattr(self, "mx", None)
        if mx and T > 32 and out_dtype == torch.bfloat16 and w.data_ptr() in mx:
            return self._mx_linear(x.contiguous(), mx[w.data_ptr()])
        out = torch.empty(x.shape[0], w.shape[0], dtype=out_dtype, device=x.device)
        if T <= 32 and self.small_decode and N % 16 == 0 and K % 32 == 0 and N * K * 2 < (48 << 20) and x.is_contiguous():
            # a few rows against a small weight matrix (decode projections): the weight-streaming mma.sync kernel
            # (measured: faster than the narrow tcgen05 tiles up to 32 rows, slower at 64)
            self.C.small_gemv(x, None, 0.0, w, None, out, self.status)
            self.launches += 1
            return out
        return self._gemm(x, w, out)

    def linear_dgrad(self, dy, w):
        dx = torch.empty(dy.shape[0], w.shape[1], dtype=torch.bfloat16, device=dy.device)
        return self._gemm(dy, w, dx, False, True)

    def linear_wgrad(self, dy, x, dw):
        """dw [N,K] += dy[M,N]^T . x[M,K]"""
        return self._gemm(dy, x, dw, True, True, True)

    def check_status(self) -> None:
        code = int(self.status.item())
        if code != 0:
            self.status.zero_()
            raise RuntimeError(f"a miles_b200 kernel reported error status {code} (bounded wait expired)")

    # ------------------------------------------------------------------ MoE block
    def _route(self, h2, router_w, replay_ids, bias=None):
        cfg, C = self.cfg, self.C
        logits = self.linear(h2, router_w, torch.float32)
        if cfg.router_score == "sigmoid":
            # GLM-4.5 / DeepSeek-V3 routing: a [T, E] problem, done with framework ops (ops/reference.py); what the
            # backward needs is the logits, kept in the place of the softmax probabilities
            from ..ops.reference import router_sigmoid_topk

            ids, w, _ = router_sigmoid_topk(logits, cfg.moe_top_k, cfg.norm_topk_prob, bias, cfg.routed_scaling_factor,
                                            cfg.n_group, cfg.topk_group, replay_ids)
            self.launches += 8
            return ids.contiguous(), w.contiguous(), logits
        rid = replay_ids.contiguous() if replay_ids is not None else None
        ids, w, probs = C.moe_router_topk(logits, rid, cfg.moe_top_k, cfg.norm_topk_prob, True)
        self.launches += 1
        return ids, w, probs

    def _permute_plan(self, ids, E_local, align: int = 1) -> MoeCtx:
        """Expert-sorted row layout. ``align`` pads every expert's rows: 64 when weight gradients will be taken
        (the wgrad contraction runs in 64-row blocks that must not straddle experts), 1 for inference."""
        T, K = ids.shape
        max_rows = max(T * K + E_local * (align - 1), 1)
        counts, offsets, dest, src, tg, nt = self.C.moe_build_permutation(ids, E_local, max_rows, align)
        self.launches += 3
        ctx = MoeCtx(ids, None, None, offsets, dest, src, tg, nt, max_rows)
        ctx.align = align
        return ctx

    def _experts_fwd(self, xp, plan: MoeCtx, w1, w2, keep: bool, scatter=None):
        """``scatter = (row_ptrs, ctrl, flag_ptrs, rank)``: the second GEMM stores every output row at its own
        address (the expert-parallel return buffers of the ranks the tokens came from) and raises their flags."""
        C = self.C
        I2 = w1.shape[1]
        mx = getattr(self, "mx", None)
        if mx and not keep and scatter is None and w1.data_ptr() in mx and w2.data_ptr() in mx and plan.align == 128:
            # rows of xp past the live tiles are never written: the per-tensor scale of NVFP4 must not look at them
            gu = self._mx_linear(xp, mx[w1.data_ptr()], plan.tile_group, plan.num_tiles, I2, getattr(plan, "amax_in", None))
            act = C.swiglu_fwd(gu)
            yp = self._mx_linear(act, mx[w2.data_ptr()], plan.tile_group, plan.num_tiles, w2.shape[1])
            self.launches += 1
            return None, None, yp
        gu = torch.empty(plan.max_rows, I2, dtype=torch.bfloat16, device=xp.device)
        C.grouped_gemm_rows(xp, w1, gu, plan.tile_group, plan.num_tiles, False, False, 0, self.status)
        act = C.swiglu_fwd(gu)
        yp = torch.empty(plan.max_rows if scatter is None else 1, w2.shape[1], dtype=torch.bfloat16, device=xp.device)
        if scatter is None:
            C.grouped_gemm_rows(act, w2, yp, plan.tile_group, plan.num_tiles, False, False, 0, self.status)
        else:
            C.grouped_gemm_rows(act, w2, yp.expand(plan.max_rows, -1), plan.tile_group, plan.num_tiles, False, False, 0,
                                self.status, scatter[0], scatter[1], scatter[2], scatter[3])
        self.launches += 3
        return (gu, act, yp) if keep else (None, None, yp)

    def moe_forward(self, i, h2, replay_ids=None, record=None, keep=False, residual=None):
        cfg, P, C = self.cfg, self.store.params, self.C
        p = f"layers.{i}.moe."
        ids, w, probs = self._route(h2, P[p + "router.weight"], replay_ids, P.get(p + "router.bias"))
        if record is not None:
            record.append(ids)
        if cfg.shared_expert_ffn and not (keep and residual is None):  # (the backward's recompute does not need the output)
            # the shared expert sees every token: its output joins the residual that the combine adds
            sh_gu = self.linear(h2, P[p + "shared.gate_up.weight"])
            sh_y = self.linear(C.swiglu_fwd(sh_gu), P[p + "shared.down.weight"])
            if cfg.shared_expert_gate:  # one sigmoid gate value per token (a [T, H] x [H] product: framework ops)
                g = torch.sigmoid(h2.float() @ P[p + "shared.gate.weight"].float().t())
                sh_y = (sh_y.float() * g).to(sh_y.dtype)
                self.launches += 3
            residual = sh_y.add_(residual) if residual is not None else sh_y
            self.launches += 3
        if self.ep is not None:
            return self.ep.moe_forward(self, i, h2, ids, w, probs, keep, residual)
        use_mx = bool(getattr(self, "mx", None)) and not keep and h2.shape[0] > 32
        plan = self._permute_plan(ids, cfg.num_experts, 64 if keep else (128 if use_mx else 1))
        plan.w, plan.probs = w, probs
        xp = C.moe_permute(h2, plan.src, plan.num_tiles, cfg.moe_top_k)
        if use_mx and self.mx_kind == "nvfp4":
            plan.amax_in = C.absmax(h2.contiguous())  # the permuted rows hold exactly these values
        gu, act, yp = self._experts_fwd(xp, plan, P[p + "w1"], P[p + "w2"], keep)
        y = C.moe_combine(yp, plan.dest, w, h2.shape[0], cfg.moe_top_k, residual)
        self.launches += 2
        saved = (plan, xp, gu, act, yp) if keep else None
        return y, saved

    def moe_backward(self, i, h2, dy, saved):
        """Returns dh2 (gradient wrt the normalised MoE input); accumulates router / expert weight grads."""
        cfg, P, G, C = self.cfg, self.store.params, self.store.grads, self.C
        p = f"layers.{i}.moe."
        if self.ep is not None:
            dh2 = self.ep.moe_backward(self, i, h2, dy, saved)
            return self._shared_expert_bwd(i, h2, dy, dh2)
        plan, xp, gu, act, yp = saved
        w1, w2 = P[p + "w1"], P[p + "w2"]
        dyp, dw = C.moe_combine_bwd(dy, yp, plan.src, plan.num_tiles, plan.w)
        dxp = self._experts_bwd(dyp, xp, gu, act, plan, w1, w2, G[p + "w1"], G[p + "w2"])
        dh2 = C.moe_combine(dxp, plan.dest, None, h2.shape[0], cfg.moe_top_k)
        self.launches += 2
        dh2 = self._router_bwd(i, h2, dh2, plan.probs, plan.ids, plan.w, dw)
        return self._shared_expert_bwd(i, h2, dy, dh2)

    def _shared_expert_bwd(self, i, h2, dy, dh2):
        """The shared expert's part of the MoE backward (recomputed from ``h2``): weight gradients, and its input gradient
        added to ``dh2``."""
        cfg, P, G, C = self.cfg, self.store.params, self.store.grads, self.C
        if not cfg.shared_expert_ffn:
            return dh2
        p = f"layers.{i}.moe.shared."
        wgu, wd = P[p + "gate_up.weight"], P[p + "down.weight"]
        dyb = dy if dy.dtype == torch.bfloat16 else dy.to(torch.bfloat16)
        gu = self.linear(h2, wgu)
        act = C.swiglu_fwd(gu)
        if cfg.shared_expert_gate:
            # y = g * s with g = sigmoid(h2 . w_g), s the shared expert's output (recomputed): ds = g dy,
            # d(logit) = (dy . s) g (1 - g), which reaches w_g and h2
            wg = P[p + "gate.weight"]
            s = self.linear(act, wd).float()
            g = torch.sigmoid(h2.float() @ wg.float().t())
            dlogit = (dy.float() * s).sum(-1, keepdim=True) * g * (1.0 - g)
            G[p + "gate.weight"].add_((dlogit.t() @ h2.float()).to(G[p + "gate.weight"].dtype))
            dh2.add_((dlogit @ wg.float()).to(dh2.dtype))
            dyb = (dy.float() * g).to(torch.bfloat16)
            self.launches += 8
        self.linear_wgrad(dyb, act, G[p + "down.weight"])
        dgu = C.swiglu_bwd(self.linear_dgrad(dyb, wd), gu)
        self.linear_wgrad(dgu, h2, G[p + "gate_up.weight"])
        self._gemm(dgu, wgu, dh2, False, True, True)  # dh2 += dgu . W
        self.launches += 7
        return dh2

    def _experts_bwd(self, dyp, xp, gu, act, plan, w1, w2, gw1, gw2, scatter=None):
        C = self.C
        dact = torch.empty_like(act)
        C.grouped_gemm_rows(dyp, w2, dact, plan.tile_group, plan.num_tiles, True, False, 0, self.status)
        C.grouped_gemm_contr(dyp, act, gw2, plan.offsets, True, 0, self.status)
        dgu = C.swiglu_bwd(dact, gu)
        if scatter is None:
            dxp = torch.empty_like(xp)
            C.grouped_gemm_rows(dgu, w1, dxp, plan.tile_group, plan.num_tiles, True, False, 0, self.status)
        else:  # the input-gradient rows go straight back to the ranks that own the tokens
            dxp = torch.empty(1, xp.shape[1], dtype=xp.dtype, device=xp.device)
            C.grouped_gemm_rows(dgu, w1, dxp.expand(xp.shape[0], -1), plan.tile_group, plan.num_tiles, True, False, 0,
                                self.status, scatter[0], scatter[1], scatter[2], scatter[3])
        C.grouped_gemm_contr(dgu, xp, gw1, plan.offsets, True, 0, self.status)
        self.launches += 5
        return dxp

    def _router_bwd(self, i, h2, dh2, probs, ids, w, dw):
        cfg, P, G, C = self.cfg, self.store.params, self.store.grads, self.C
        p = f"layers.{i}.moe."
        if cfg.router_score == "sigmoid":
            # ``probs`` holds the router logits (see _route): differentiate the [T, E] routing function with autograd
            from ..ops.reference import router_sigmoid_topk

            with torch.enable_grad():
                lg = probs.detach().requires_grad_(True)
                _, w2, _ = router_sigmoid_topk(lg, cfg.moe_top_k, cfg.norm_topk_prob, None, cfg.routed_scaling_factor, 1, 1, ids)
                (dlogits,) = torch.autograd.grad(w2, lg, dw.to(w2.dtype))
            dlogits = dlogits.to(torch.bfloat16)
            self.launches += 10
        else:
            dlogits = C.moe_router_bwd(probs, ids, w, dw, cfg.norm_topk_prob).to(torch.bfloat16)
        self._gemm(dlogits, P[p + "router.weight"], dh2, False, True, True)
        self.linear_wgrad(dlogits, h2, G[p + "router.weight"])
        self.launches += 1
        return dh2

    # ------------------------------------------------------------------ layer forward / backward
    def _attn_qkv(self, i, x, positions, meta: Optional[InferMeta], kv_cache):
        cfg, P, C = self.cfg, self.store.params, self.C
        p = f"layers.{i}."
        h1, rstd1 = C.rmsnorm_fwd(x, None, P[p + "ln1.weight"], cfg.rms_eps)
        qkv = self.linear(h1, P[p + "attn.qkv.weight"])
        if cfg.qkv_bias:
            qkv += P[p + "attn.qkv.bias"]
        kc = vc = slots = None
        if kv_cache is not None:
            kc, vc = kv_cache[i]
            slots = meta.slot_mapping
        write_k = meta is None or meta.is_prefill
        if cfg.rope_scaling or cfg.rotary_dim:
            q, k, qr, kr = C.qk_norm_rope_fwd_scaled(qkv, P.get(p + "attn.q_norm.weight"), P.get(p + "attn.k_norm.weight"),
                                                     positions, cfg.num_q_heads, cfg.num_kv_heads, cfg.rope_theta, cfg.rms_eps,
                                                     kc, vc, slots, write_k, self._rope_table(), cfg.rotary_dim or cfg.head_dim)
        else:
            q, k, qr, kr = C.qk_norm_rope_fwd(qkv, P.get(p + "attn.q_norm.weight"), P.get(p + "attn.k_norm.weight"), positions,
                                              cfg.num_q_heads, cfg.num_kv_heads, cfg.rope_theta, cfg.rms_eps, kc, vc, slots,
                                              write_k)
        self.launches += 2
        return h1, rstd1, qkv, q, k, qr, kr

    def _rope_table(self) -> Optional[torch.Tensor]:
        """The inverse frequencies of a model with scaled rotary embeddings (fp32, on the device); None without scaling
        (the kernels then compute theta^(-d / half) themselves)."""
        if not self.cfg.rope_scaling:
            return None
        t = getattr(self, "_inv_freq", None)
        if t is None:
            from ..ops.reference import rope_inv_freq

            t = self._inv_freq = rope_inv_freq(self.cfg.rotary_dim or self.cfg.head_dim, self.cfg.rope_theta, self.cfg.rope_scaling,
                                               self.dev).contiguous()
        return t

    def _v_view(self, qkv):
        cfg = self.cfg
        return qkv.view(qkv.shape[0], cfg.num_q_heads + 2 * cfg.num_kv_heads, cfg.head_dim)[:, cfg.num_q_heads + cfg.num_kv_heads:]

    def layer_forward(self, i, x, positions, cu, max_seqlen, meta: Optional[InferMeta] = None, kv_cache=None,
                      replay_ids=None, record=None):
        """Inference/no-grad forward of one layer: returns the layer output."""
        cfg, P, C = self.cfg, self.store.params, self.C
        p = f"layers.{i}."
        if (meta is not None and not meta.is_prefill and x.shape[0] <= self.SMALL_T and replay_ids is None
                and self.small_decode and self.tp is None and not cfg.post_norms):
            # the fused few-row MoE kernels serve plain softmax routers whose expert count fits their 16-column tiles
            plain_moe = cfg.router_score == "softmax" and not cfg.shared_expert_ffn and cfg.num_experts % 16 == 0
            if (self.ep is None and plain_moe) or not cfg.layer_is_moe(i):
                return self._layer_forward_small(i, x, positions, meta, kv_cache, record)
            # expert-parallel MoE: the attention half still takes the light kernels, the experts go through the exchange
            x2 = self._attn_small(i, x, positions, meta, kv_cache)
            if getattr(self.ep, "low_latency", False) and plain_moe:
                return self.ep.moe_decode(self, i, x2, None, record)
            h2, _ = C.rmsnorm_fwd(x2, None, P[p + "ln2.weight"], cfg.rms_eps)
            self.launches += 1
            y, _ = self.moe_forward(i, h2, replay_ids, record, keep=False, residual=x2)
            return y
        h1, rstd1, qkv, q, k, _, _ = self._attn_qkv(i, x, positions, meta, kv_cache)
        scale = cfg.head_dim ** -0.5
        if meta is not None and not meta.is_prefill:
            att = torch.empty_like(q)
            B = q.shape[0]
            splits = self._decode_splits(B, meta)
            need = B * cfg.num_q_heads * splits * 130
            if self._decode_scratch is None or self._decode_scratch.numel() < need:
                self._decode_scratch = torch.empty(need, dtype=torch.float32, device=self.dev)
            kc, vc = kv_cache[i]
            C.paged_decode_attention(q, kc, vc, meta.block_table, meta.seq_lens, att, self._decode_scratch, meta.page_size,
                                     splits, scale)
            self.launches += 2
        elif meta is not None and getattr(meta, "prefix", None) is not None:
            # prefill behind a cached prefix: the keys / values of the cached tokens come from their pages, the tile
            # table gives every query tile its sequence's key range and the position of its first query
            kf, vf = meta.prefix.full_kv(k, self._v_view(qkv), *kv_cache[i])
            att, _ = self.C.flash_attn_fwd(q, kf, vf, meta.prefix.tiles, scale, self.status)
            self.launches += 5
        else:
            att, _ = self.attention(q, k, self._v_view(qkv), cu)
        h2, _, x2 = self._o_proj_ln2(i, att.view(att.shape[0], -1), x)
        if cfg.layer_is_moe(i):
            if (meta is not None and not meta.is_prefill and replay_ids is None and getattr(self.ep, "low_latency", False)
                    and x.shape[0] <= self.ep.rows and cfg.router_score == "softmax" and not cfg.shared_expert_ffn):
                return self.ep.moe_decode(self, i, x2, h2, record)
            y, _ = self.moe_forward(i, h2, replay_ids, record, keep=False, residual=x2)
            return y
        gu = self.linear(h2, P[p + "mlp.gate_up.weight"])
        self.launches += 1
        if cfg.post_norms:
            y = self.linear(C.swiglu_fwd(gu), P[p + "mlp.down.weight"])
            yn, _ = C.rmsnorm_fwd(y, None, P[p + "post_mlp_ln.weight"], cfg.rms_eps)
            self.launches += 2
            return yn.add_(x2)
        return self._row_parallel(C.swiglu_fwd(gu), P[p + "mlp.down.weight"], x2)

    def _row_parallel(self, a, w, residual):
        """``residual + a @ w^T`` for a row-parallel weight: under tensor parallelism the GEMM epilogue pushes the
        partial sums to the peers and the slots are added in rank order (one fused GEMM + all-reduce)."""
        if self.tp is not None:
            self.launches += 3
            return self.tp.linear_allreduce(a, w, residual=residual, gemm_status=self.status)
        y = self.linear(a, w)
        return y.add_(residual) if residual is not None else y

    def _o_proj_ln2(self, i, att2, x):
        """Attention output projection, residual add and the second RMSNorm: returns (h2, rstd2, x2)."""
        cfg, P, C = self.cfg, self.store.params, self.C
        p = f"layers.{i}."
        self.launches += 1
        if self.tp is not None:
            assert not cfg.post_norms, "models with sandwich norms run without tensor parallelism"
            x2 = self._row_parallel(att2, P[p + "attn.o.weight"], x)
            h2, rstd2 = C.rmsnorm_fwd(x2, None, P[p + "ln2.weight"], cfg.rms_eps)
            return h2, rstd2, x2
        o = self.linear(att2, P[p + "attn.o.weight"])
        if cfg.post_norms:
            # sandwich norm (GLM-4 dense): the attention output is normalised before it joins the residual stream; the
            # backward's recompute picks the un-normalised output and its statistics up from here
            on, rstd_pa = C.rmsnorm_fwd(o, None, P[p + "post_attn_ln.weight"], cfg.rms_eps)
            self._post_attn_saved = (o, rstd_pa)
            self.launches += 1
            return C.rmsnorm_fwd(on, x, P[p + "ln2.weight"], cfg.rms_eps)
        return C.rmsnorm_fwd(o, x, P[p + "ln2.weight"], cfg.rms_eps)

    def _col_parallel_dgrad(self, dy, w):
        """Input gradient of a column-parallel weight: partial over the tensor-parallel ranks, so all-reduced."""
        if self.tp is not None:
            self.launches += 3
            return self.tp.linear_allreduce(dy, w, b_mn=True, gemm_status=self.status)
        return self.linear_dgrad(dy, w)

    SMALL_T = 8  # decode steps with at most this many rows take the weight-streaming kernels

    def _attn_small(self, i, x, positions, meta: InferMeta, kv_cache):
        """Attention half of a decode layer for at most 8 rows: returns ``x + attention(x)`` (RMSNorm folded into the
        qkv projection, residual folded into the output projection)."""
        cfg, P, C = self.cfg, self.store.params, self.C
        p = f"layers.{i}."
        T, dev = x.shape[0], x.device
        wqkv = P[p + "attn.qkv.weight"]
        qkv = torch.empty(T, wqkv.shape[0], dtype=torch.bfloat16, device=dev)
        C.small_gemv(x, P[p + "ln1.weight"], cfg.rms_eps, wqkv, None, qkv, self.status)
        if cfg.qkv_bias:
            qkv += P[p + "attn.qkv.bias"]
        kc, vc = kv_cache[i]
        if cfg.rope_scaling or cfg.rotary_dim:
            q, _, _, _ = C.qk_norm_rope_fwd_scaled(qkv, P.get(p + "attn.q_norm.weight"), P.get(p + "attn.k_norm.weight"),
                                                   positions, cfg.num_q_heads, cfg.num_kv_heads, cfg.rope_theta, cfg.rms_eps,
                                                   kc, vc, meta.slot_mapping, False, self._rope_table(),
                                                   cfg.rotary_dim or cfg.head_dim)
        else:
            q, _, _, _ = C.qk_norm_rope_fwd(qkv, P.get(p + "attn.q_norm.weight"), P.get(p + "attn.k_norm.weight"), positions,
                                            cfg.num_q_heads, cfg.num_kv_heads, cfg.rope_theta, cfg.rms_eps, kc, vc,
                                            meta.slot_mapping, False)
        att = torch.empty_like(q)
        splits = self._decode_splits(T, meta)
        need = T * cfg.num_q_heads * splits * 130
        if self._decode_scratch is None or self._decode_scratch.numel() < need:
            self._decode_scratch = torch.empty(need, dtype=torch.float32, device=dev)
        C.paged_decode_attention(q, kc, vc, meta.block_table, meta.seq_lens, att, self._decode_scratch, meta.page_size,
                                 splits, cfg.head_dim ** -0.5)
        x2 = torch.empty_like(x)
        C.small_gemv(att.view(T, -1), None, cfg.rms_eps, P[p + "attn.o.weight"], x, x2, self.status)
        self.launches += 6
        return x2

    def _layer_forward_small(self, i, x, positions, meta: InferMeta, kv_cache, record=None):
        """Decode forward of one layer for at most 8 rows: 8-9 light launches instead of 14-15, the two RMSNorms
        folded into the projections that consume them, no expert permutation (per-expert pair lists)."""
        cfg, P, C = self.cfg, self.store.params, self.C
        p = f"layers.{i}."
        T, dev = x.shape[0], x.device
        x2 = self._attn_small(i, x, positions, meta, kv_cache)
        ln2 = P[p + "ln2.weight"]
        if cfg.layer_is_moe(i):
            E, K = cfg.num_experts, cfg.moe_top_k
            w1, w2 = P[p + "moe.w1"], P[p + "moe.w2"]
            ids = torch.empty(T, K, dtype=torch.int32, device=dev)
            w = torch.empty(T, K, dtype=torch.float32, device=dev)
            lists = torch.empty(1 + E + E + 8 * E, dtype=torch.int32, device=dev)
            active, pc, pl = lists[:1 + E], lists[1 + E:1 + 2 * E], lists[1 + 2 * E:]
            logits = torch.empty(T, E, dtype=torch.float32, device=dev)
            C.small_gemv(x2, ln2, cfg.rms_eps, P[p + "moe.router.weight"], None, logits, self.status)
            C.router_small(logits, K, cfg.norm_topk_prob, ids, w, active, pc, pl)
            if record is not None:
                record.append(ids)
            max_active = min(E, T * K)
            act = torch.empty(T * K, w1.shape[1], dtype=torch.bfloat16, device=dev)  # gate | up; SwiGLU happens in the consumer
            C.moe_small_up(x2, ln2, cfg.rms_eps, w1, active, pc, pl, max_active, K, act, self.status)
            yp = torch.empty(T * K, x.shape[1], dtype=torch.bfloat16, device=dev)
            C.moe_small_down(act, w2, active, pc, pl, max_active, yp, self.status)
            if self._ident is None or self._ident.numel() < T * K:
                self._ident = torch.arange(self.SMALL_T * K, dtype=torch.int32, device=dev)
            y = C.moe_combine(yp, self._ident[:T * K], w, T, K, x2)
            self.launches += 5
            return y
        wgu = P[p + "mlp.gate_up.weight"]
        gu = torch.empty(T, wgu.shape[0], dtype=torch.bfloat16, device=dev)
        C.small_gemv(x2, ln2, cfg.rms_eps, wgu, None, gu, self.status)
        y = torch.empty_like(x)
        C.small_gemv(C.swiglu_fwd(gu), None, cfg.rms_eps, P[p + "mlp.down.weight"], x2, y, self.status)
        self.launches += 3
        return y

    def _decode_splits(self, B: int, meta: InferMeta) -> int:
        ctas = B * self.cfg.num_kv_heads
        return max(1, min(16, (148 * 3) // max(ctas, 1)))

    def layer_backward(self, i, x, dy, positions, cu, max_seqlen, replay_ids=None):
        """Recompute layer i from its input ``x`` and back-propagate ``dy``; returns dx."""
        cfg, P, G, C = self.cfg, self.store.params, self.store.grads, self.C
        p = f"layers.{i}."
        scale = cfg.head_dim ** -0.5
        # ---- recompute forward, keeping what the backward needs
        h1, rstd1, qkv, q, k, qr, kr = self._attn_qkv(i, x, positions, None, None)
        v = self._v_view(qkv)
        att, lse = self.attention(q, k, v, cu)
        att2 = att.view(att.shape[0], -1)
        h2, rstd2, x2 = self._o_proj_ln2(i, att2, x)
        post_attn = getattr(self, "_post_attn_saved", None) if cfg.post_norms else None
        self._post_attn_saved = None
        is_moe = cfg.layer_is_moe(i)
        assert not (is_moe and cfg.post_norms), "sandwich norms are wired for dense MLP layers"
        if is_moe:
            _, saved = self.moe_forward(i, h2, replay_ids, None, keep=True)
        else:
            gu = self.linear(h2, P[p + "mlp.gate_up.weight"])
            act = C.swiglu_fwd(gu)
            self.launches += 1
        # ---- backward: MLP / MoE
        if is_moe:
            dh2 = self.moe_backward(i, h2, dy, saved)
            del saved
        else:
            dyy = dy
            if cfg.post_norms:  # through the norm on the MLP output (its input is recomputed)
                y = self.linear(act, P[p + "mlp.down.weight"])
                _, rstd_pm = C.rmsnorm_fwd(y, None, P[p + "post_mlp_ln.weight"], cfg.rms_eps)
                dyy = C.rmsnorm_bwd(dy, y, P[p + "post_mlp_ln.weight"], rstd_pm, None, G[p + "post_mlp_ln.weight"], True)
                self.launches += 3
            dact = self.linear_dgrad(dyy, P[p + "mlp.down.weight"])
            self.linear_wgrad(dyy, act, G[p + "mlp.down.weight"])
            dgu = C.swiglu_bwd(dact, gu)
            dh2 = self._col_parallel_dgrad(dgu, P[p + "mlp.gate_up.weight"])
            self.linear_wgrad(dgu, h2, G[p + "mlp.gate_up.weight"])
            self.launches += 1
        # ---- ln2 (residual gradient dy flows straight through x2)
        dx2 = C.rmsnorm_bwd(dh2, x2, P[p + "ln2.weight"], rstd2, dy, G[p + "ln2.weight"], True)
        self.launches += 2
        # ---- attention output projection
        do = dx2
        if cfg.post_norms:  # through the norm on the attention output
            o, rstd_pa = post_attn
            do = C.rmsnorm_bwd(dx2, o, P[p + "post_attn_ln.weight"], rstd_pa, None, G[p + "post_attn_ln.weight"], True)
            self.launches += 1
        datt = self.linear_dgrad(do, P[p + "attn.o.weight"])
        self.linear_wgrad(do, att2, G[p + "attn.o.weight"])
        dq, dk, dv = self.attention_backward(q, k, v, att, datt.view_as(att), lse, cu)
        if cfg.rope_scaling or cfg.rotary_dim:
            dqkv = C.qk_norm_rope_bwd_scaled(dq, dk, dv, qkv, P.get(p + "attn.q_norm.weight"),
                                             P.get(p + "attn.k_norm.weight"), positions, qr, kr, G.get(p + "attn.q_norm.weight"),
                                             G.get(p + "attn.k_norm.weight"), cfg.num_q_heads, cfg.num_kv_heads, cfg.rope_theta,
                                             self._rope_table(), cfg.rotary_dim or cfg.head_dim)
        else:
            dqkv = C.qk_norm_rope_bwd(dq, dk, dv, qkv, P.get(p + "attn.q_norm.weight"),
                                      P.get(p + "attn.k_norm.weight"), positions, qr, kr, G.get(p + "attn.q_norm.weight"),
                                      G.get(p + "attn.k_norm.weight"), cfg.num_q_heads, cfg.num_kv_heads, cfg.rope_theta)
        self.launches += 1
        if cfg.qkv_bias:
            G[p + "attn.qkv.bias"].add_(dqkv.float().sum(0).to(G[p + "attn.qkv.bias"].dtype))
        dh1 = self._col_parallel_dgrad(dqkv, P[p + "attn.qkv.weight"])
        self.linear_wgrad(dqkv, h1, G[p + "attn.qkv.weight"])
        dx = C.rmsnorm_bwd(dh1, x, P[p + "ln1.weight"], rstd1, dx2, G[p + "ln1.weight"], True)
        self.launches += 2
        return dx

    # ------------------------------------------------------------------ whole-model passes
    @torch.no_grad()
    def forward_hidden(self, tokens, positions, cu_seqlens, meta: Optional[InferMeta] = None, kv_cache=None,
                       replay: Optional[torch.Tensor] = None, record: Optional[list] = None, max_seqlen: int = 0,
                       save_inputs: Optional[list] = None, x_in: Optional[torch.Tensor] = None):
        """Runs this pipeline stage's layers (all of them without pipeline parallelism). The first stage embeds
        ``tokens``, later stages continue from ``x_in``; every stage but the last returns the raw hidden states that
        the next stage consumes, the last one applies the final norm."""
        cfg, P, C = self.cfg, self.store.params, self.C
        begin = getattr(self.store, "begin_pass", None)
        if begin is not None:
            begin()  # a sharded store materialises units per pass
        lo, hi = self.store.layer_range
        x = P["embed.weight"][tokens.long()] if self.store.is_first_stage else x_in
        if not max_seqlen and cu_seqlens is not None:
            max_seqlen = int((cu_seqlens[1:] - cu_seqlens[:-1]).max().item())
        moe_idx = sum(cfg.layer_is_moe(j) for j in range(lo))  # replay columns are indexed over the whole model
        for i in range(lo, hi):
            if save_inputs is not None:
                save_inputs.append(x)
            rid = None
            if cfg.layer_is_moe(i):
                if replay is not None:
                    rid = replay[:, moe_idx]
                moe_idx += 1
            x = self.layer_forward(i, x, positions, cu_seqlens, max_seqlen, meta, kv_cache, rid, record)
        if save_inputs is not None:
            save_inputs.append(x)
        if not self.store.is_last_stage:
            return x
        h, _ = C.rmsnorm_fwd(x, None, P["final_norm.weight"], cfg.rms_eps)
        self.launches += 1
        return h

    @torch.no_grad()
    def _trunk_backward(self, inputs, x_last, h, rows, dhr, tokens, positions, cu_seqlens, max_seqlen, replay):
        """Back-propagate ``dhr`` (gradient wrt the final-normed hidden rows) through the norm, layers and embedding."""
        cfg, P, G, C = self.cfg, self.store.params, self.store.grads, self.C
        dh = torch.zeros_like(h)
        dh.index_add_(0, rows, dhr.to(h.dtype))
        _, rstd = C.rmsnorm_fwd(x_last, None, P["final_norm.weight"], cfg.rms_eps)
        dx = C.rmsnorm_bwd(dh, x_last, P["final_norm.weight"], rstd, None, G["final_norm.weight"], True)
        self.launches += 3
        del dh
        return self.layers_backward(inputs, dx, tokens, positions, cu_seqlens, max_seqlen, replay)

    @torch.no_grad()
    def layers_backward(self, inputs, dx, tokens, positions, cu_seqlens, max_seqlen, replay):
        """Backward through this stage's layers: ``inputs[j]`` is the saved input of local layer ``j``, ``dx`` the
        gradient of the stage's output. Returns the gradient of the stage's input (on the first stage it has been
        added into the embedding gradient) and keeps it in ``self.last_dx_in``."""
        cfg, G = self.cfg, self.store.grads
        lo, hi = self.store.layer_range
        moe_layers = [i for i in range(cfg.num_layers) if cfg.layer_is_moe(i)]
        for i in reversed(range(lo, hi)):
            rid = replay[:, moe_layers.index(i)] if (replay is not None and cfg.layer_is_moe(i)) else None
            dx = self.layer_backward(i, inputs[i - lo], dx, positions, cu_seqlens, max_seqlen, rid)
            inputs[i - lo] = None
        if self.store.is_first_stage:
            G["embed.weight"].index_add_(0, tokens.long(), dx.to(G["embed.weight"].dtype))
        self.last_dx_in = dx
        return dx

    def forward_backward_hidden(self, tokens, positions, cu_seqlens, row_index, head_fn, replay=None, max_seqlen: int = 0,
                                x_in: Optional[torch.Tensor] = None):
        """Generic head: ``head_fn(hidden_rows_fp32_leaf) -> (loss, metrics)`` (e.g. a value head); the trunk is
        back-propagated with the gradient autograd computes for the hidden rows."""
        assert self.store.grads, "allocate_grads() must be called before training"
        if not max_seqlen:
            max_seqlen = int((cu_seqlens[1:] - cu_seqlens[:-1]).max().item())
        inputs: list = []
        h = self.forward_hidden(tokens, positions, cu_seqlens, replay=replay, max_seqlen=max_seqlen, save_inputs=inputs, x_in=x_in)
        x_last = inputs.pop()
        rows = row_index.long()
        leaf = h[rows].float().detach().requires_grad_(True)
        with torch.enable_grad():
            loss, metrics = head_fn(leaf)
            loss.backward()
        self._trunk_backward(inputs, x_last, h, rows, leaf.grad, tokens, positions, cu_seqlens, max_seqlen, replay)
        return loss.detach(), metrics

    @torch.no_grad()
    def logits(self, hidden_rows, out_dtype=torch.float32):
        return self.linear(hidden_rows.contiguous(), self.store.lm_head(), out_dtype)

    @torch.no_grad()
    def logprobs_entropy(self, hidden_rows, targets, inv_temp: float, chunk: int = 0, keep_stats: bool = False):
        C = self.C
        chunk = chunk or self.lm_chunk
        n = hidden_rows.shape[0]
        lp = torch.empty(n, dtype=torch.float32, device=self.dev)
        ent = torch.empty_like(lp)
        lse = torch.empty_like(lp) if keep_stats else None
        px = torch.empty_like(lp) if keep_stats else None
        tg = targets.to(torch.int32).contiguous()
        for a in range(0, n, chunk):
            b = min(a + chunk, n)
            lg = self.logits(hidden_rows[a:b])
            l1, e1, s1, p1 = C.logprob_entropy_fwd(lg, tg[a:b], inv_temp)
            self.launches += 1
            lp[a:b], ent[a:b] = l1, e1
            if keep_stats:
                lse[a:b], px[a:b] = s1, p1
        return (lp, ent, lse, px) if keep_stats else (lp, ent)

    @torch.no_grad()
    def forward_logprobs(self, tokens, positions, cu_seqlens, row_index, targets, inv_temp, replay=None, record=None,
                         max_seqlen: int = 0, x_in: Optional[torch.Tensor] = None):
        h = self.forward_hidden(tokens, positions, cu_seqlens, replay=replay, record=record, max_seqlen=max_seqlen, x_in=x_in)
        return self.logprobs_entropy(h[row_index.long()], targets, inv_temp)

    def forward_backward(self, tokens, positions, cu_seqlens, row_index, targets, inv_temp, loss_fn, replay=None,
                         max_seqlen: int = 0, chunk: int = 0, x_in: Optional[torch.Tensor] = None):
        """One micro-batch: forward, ``loss_fn(logprobs, entropy) -> (loss, metrics)``, backward into the grad buffers.
        On the last pipeline stage ``x_in`` is the activation received from the previous stage and ``self.last_dx_in``
        afterwards holds the gradient to send back."""
        cfg, P, G, C = self.cfg, self.store.params, self.store.grads, self.C
        assert G, "allocate_grads() must be called before training"
        chunk = chunk or self.lm_chunk
        if not max_seqlen:
            max_seqlen = int((cu_seqlens[1:] - cu_seqlens[:-1]).max().item())
        inputs: list[torch.Tensor] = []
        h = self.forward_hidden(tokens, positions, cu_seqlens, replay=replay, max_seqlen=max_seqlen, save_inputs=inputs, x_in=x_in)
        x_last = inputs.pop()  # input of the final norm
        rows = row_index.long()
        hr = h[rows].contiguous()
        tg = targets.to(torch.int32).contiguous()
        with torch.no_grad():
            lp, ent, lse, px = self.logprobs_entropy(hr, tg, inv_temp, chunk, keep_stats=True)
        lp_leaf, ent_leaf = lp.detach().requires_grad_(True), ent.detach().requires_grad_(True)
        with torch.enable_grad():
            loss, metrics = loss_fn(lp_leaf, ent_leaf)
            grads = torch.autograd.grad(loss, (lp_leaf, ent_leaf), allow_unused=True)
        dlp = grads[0].float().contiguous() if grads[0] is not None else torch.zeros_like(lp)
        dent = grads[1].float().contiguous() if grads[1] is not None else None
        with torch.no_grad():
            # ---- LM head backward, chunked: recompute logits, turn them into dlogits in place
            W = self.store.lm_head()
            gW = G["embed.weight"] if cfg.tie_embeddings else G["lm_head.weight"]
            dhr = torch.empty_like(hr)
            for a in range(0, hr.shape[0], chunk):
                b = min(a + chunk, hr.shape[0])
                lg = self.logits(hr[a:b])
                dl = C.logprob_entropy_bwd(lg, tg[a:b], lse[a:b].contiguous(), px[a:b].contiguous(), dlp[a:b].contiguous(),
                                           dent[a:b].contiguous() if dent is not None else None, inv_temp)
                del lg
                self._gemm(dl, W, dhr[a:b], False, True)
                self.linear_wgrad(dl, hr[a:b], gW)
                self.launches += 1
            self._trunk_backward(inputs, x_last, h, rows, dhr, tokens, positions, cu_seqlens, max_seqlen, replay)
        return loss.detach(), metrics, lp.detach(), ent.detach()
