"""Expert parallelism: tokens stay with their data-parallel rank for attention, routed rows travel to the
rank that owns the expert and come back (all-to-all dispatch / combine around the grouped expert GEMMs).

Two transports:

* ``fused=True``  — in-kernel NVLink stores into the owners' symmetric receive regions with flag
  signalling (``csrc/ep_comm.cu``); device-side epochs make the sequence CUDA-graph capturable, which the
  decode path needs.
* ``fused=False`` — ``torch.distributed.all_to_all_single`` over NCCL with host-synchronised split sizes:
  the baseline every fused number is reported against.

Both are lockstep collectives: every EP rank must run the same sequence of MoE layers.
Reference: Megatron's alltoall token dispatcher (scripts/models/qwen3-30B-A3B.py:29-41).
"""
from __future__ import annotations


import torch
import torch.distributed as dist

from ..ops import _ext
from .symm import SymmetricRegion


class ExpertParallel:
    def __init__(self, cfg, ps, fused: bool = True, max_tokens: int = 32768, fused_epilogue: bool = True):
        self.cfg, self.ps = cfg, ps
        self.group, self.rank, self.n = ps.ep.group, ps.ep.rank, ps.ep.size
        self.el = cfg.num_experts // self.n
        self.fused = fused and ps.device.type == "cuda"
        # the GEMM that produces the expert outputs (or input gradients) stores them straight into the source ranks'
        # return buffers; off = a separate copy kernel after the GEMM (kept for comparison)
        self.fused_epilogue = self.fused and fused_epilogue
        self.dev = ps.device
        self.C = _ext.load(required=True) if self.dev.type == "cuda" else None
        self.K, self.H = cfg.moe_top_k, cfg.hidden_size
        self.max_entries = max_tokens * self.K
        self.cap = min(self.max_entries, int(self.max_entries / self.n * 2) + 1024)
        self.bytes_dispatched = 0
        if self.fused:
            self._setup_symmetric()

    # ------------------------------------------------------------------ symmetric buffers
    def _setup_symmetric(self) -> None:
        n, cap, H = self.n, self.cap, self.H
        nbytes = n * cap * H * 2 + n * cap * 8 + self.max_entries * H * 2 + 64 * 1024
        self.region = SymmetricRegion(nbytes, self.group, self.rank, n, self.dev)
        self.xrecv, self.p_xrecv = self.region.carve((n * cap, H), torch.bfloat16)
        self.meta, self.p_meta = self.region.carve((n * cap, 2), torch.int32)
        self.counts, self.p_counts = self.region.carve((n,), torch.int32)
        self.flags, self.p_flags = self.region.carve((n,), torch.int64)
        self.yback, self.p_yback = self.region.carve((self.max_entries, H), torch.bfloat16)
        self.flags2, self.p_flags2 = self.region.carve((n,), torch.int64)
        self.ctrl = torch.zeros(8, dtype=torch.int64, device=self.dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.dev)
        self.identity = torch.arange(self.max_entries, dtype=torch.int32, device=self.dev)
        self.big_tiles = torch.tensor([1 << 20, 1 << 30], dtype=torch.int32, device=self.dev)
        self.pos_in_cap = torch.arange(cap, dtype=torch.int32, device=self.dev)[None, :]
        self._peers = (self.p_xrecv, self.p_meta, self.p_counts, self.p_flags, self.p_yback, self.p_flags2)

    def check_status(self) -> None:
        if self.fused:
            code = int(self.status.item())
            if code:
                self.status.zero_()
                raise RuntimeError(f"expert-parallel exchange reported error {code} (5 = peer wait expired, 7 = capacity overflow)")

    # ------------------------------------------------------------------ fused transport
    def _send(self, rows, ids_flat, route, row_div):
        C = self.C
        counts_r, offsets_r, dest_r = route
        C.ep_dispatch(rows, ids_flat, dest_r, offsets_r, counts_r, *self._peers, self.rank, self.el, row_div, self.cap,
                      self.ctrl, self.status)
        C.ep_wait(self.flags, self.n, self.ctrl, 1, self.status)
        self.bytes_dispatched += rows.shape[-1] * 2 * ids_flat.numel()

    def _recv_plan(self, model, align: int = 1):
        """Group the received rows by local expert (rows beyond each source's count are ignored)."""
        n, cap = self.n, self.cap
        valid = self.pos_in_cap < self.counts[:, None]
        ids_recv = torch.where(valid, self.meta.view(n, cap, 2)[:, :, 0], torch.full_like(self.pos_in_cap, -1))
        return model._permute_plan(ids_recv.reshape(n * cap, 1).contiguous(), self.el, align)

    def _scatter_args(self, plan):
        """Arguments that turn the producing GEMM's epilogue into the return transfer (rows stored straight into the
        source ranks' return regions over NVLink, flags raised by the last CTA)."""
        ptrs = self.C.ep_row_ptrs(plan.src, self.meta, *self._peers, self.cap, self.H)
        return ptrs, self.ctrl, self.p_flags2, self.rank

    def _await_return(self, n_entries):
        self.C.ep_wait(self.flags2, self.n, self.ctrl, 3, self.status)
        return self.yback[:n_entries]

    def _return(self, rows_perm, plan, n_entries):
        C = self.C
        C.ep_return(rows_perm, plan.dest, self.meta, self.counts, *self._peers, self.rank, self.cap, self.ctrl, self.status)
        C.ep_wait(self.flags2, self.n, self.ctrl, 3, self.status)
        return self.yback[:n_entries]

    def _route(self, ids):
        T, K = ids.shape
        ids_rank = torch.div(ids, self.el, rounding_mode="floor").to(torch.int32).contiguous()
        counts_r, offsets_r, dest_r, _, _, _ = self.C.moe_build_permutation(ids_rank, self.n, T * K, 1)
        return counts_r, offsets_r, dest_r

    def moe_forward(self, model, i, h2, ids, w, probs, keep: bool, residual=None):
        if not self.fused:
            y, saved = self._moe_forward_nccl(model, i, h2, ids, w, probs, keep)
            return (y if residual is None else y.add_(residual)), saved
        cfg, P, C = self.cfg, model.store.params, self.C
        p = f"layers.{i}.moe."
        T, K = ids.shape
        n_entries = T * K
        assert n_entries <= self.max_entries, f"{T} tokens exceed the expert-parallel buffer ({self.max_entries // K})"
        route = self._route(ids)
        ids_flat = ids.reshape(-1)
        self._send(h2, ids_flat, route, K)
        plan = self._recv_plan(model, 64 if keep else 1)
        xp = C.moe_permute(self.xrecv, plan.src, plan.num_tiles, 1)
        if self.fused_epilogue:
            gu, act, _ = model._experts_fwd(xp, plan, P[p + "w1"], P[p + "w2"], keep, scatter=self._scatter_args(plan))
            yslot = self._await_return(n_entries)
        else:
            gu, act, yp = model._experts_fwd(xp, plan, P[p + "w1"], P[p + "w2"], keep)
            yslot = self._return(yp, plan, n_entries)
        y = C.moe_combine(yslot, self.identity[:n_entries], w, T, K, residual)
        model.launches += 8
        saved = None
        if keep:
            saved = dict(plan=plan, xp=xp, gu=gu, act=act, route=route, ids=ids, w=w, probs=probs, yslot=yslot.clone())
        return y, saved

    def moe_backward(self, model, i, h2, dy, saved):
        if not self.fused:
            return self._moe_backward_nccl(model, i, h2, dy, saved)
        cfg, P, G, C = self.cfg, model.store.params, model.store.grads, self.C
        p = f"layers.{i}.moe."
        ids, w, plan = saved["ids"], saved["w"], saved["plan"]
        T, K = ids.shape
        n_entries = T * K
        dy_slot, dw = C.moe_combine_bwd(dy, saved["yslot"], self.identity[:n_entries], self.big_tiles, w)
        self._send(dy_slot, ids.reshape(-1), saved["route"], 1)
        dyp = C.moe_permute(self.xrecv, plan.src, plan.num_tiles, 1)
        if self.fused_epilogue:
            model._experts_bwd(dyp, saved["xp"], saved["gu"], saved["act"], plan, P[p + "w1"], P[p + "w2"],
                               G[p + "w1"], G[p + "w2"], scatter=self._scatter_args(plan))
            dslot = self._await_return(n_entries)
        else:
            dxp = model._experts_bwd(dyp, saved["xp"], saved["gu"], saved["act"], plan, P[p + "w1"], P[p + "w2"],
                                     G[p + "w1"], G[p + "w2"])
            dslot = self._return(dxp, plan, n_entries)
        dh2 = C.moe_combine(dslot, self.identity[:n_entries], None, T, K)
        model.launches += 8
        return model._router_bwd(i, h2, dh2, saved["probs"], ids, w, dw)

    # ------------------------------------------------------------------ NCCL baseline transport
    def _exchange_nccl(self, rows_sorted, send_counts, recv_counts):
        out = torch.empty(int(sum(recv_counts)), rows_sorted.shape[1], dtype=rows_sorted.dtype, device=rows_sorted.device)
        dist.all_to_all_single(out, rows_sorted, recv_counts, send_counts, group=self.group)
        return out

    def _nccl_plan(self, ids):
        T, K = ids.shape
        flat = ids.reshape(-1).long()
        dest = torch.div(flat, self.el, rounding_mode="floor")
        order = torch.argsort(dest, stable=True)
        send_counts = torch.bincount(dest, minlength=self.n)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        sc, rc = send_counts.tolist(), recv_counts.tolist()
        le_sorted = (flat[order] % self.el).to(torch.int32)
        le_recv = self._exchange_nccl(le_sorted[:, None].contiguous(), sc, rc)
        return order, sc, rc, le_recv

    def _moe_forward_nccl(self, model, i, h2, ids, w, probs, keep):
        cfg, P, C = self.cfg, model.store.params, self.C
        p = f"layers.{i}.moe."
        T, K = ids.shape
        order, sc, rc, le_recv = self._nccl_plan(ids)
        rows = h2[torch.div(order, K, rounding_mode="floor")]
        xr = self._exchange_nccl(rows.contiguous(), sc, rc)
        plan = model._permute_plan(le_recv.contiguous(), self.el, 64 if keep else 1)
        xp = C.moe_permute(xr, plan.src, plan.num_tiles, 1)
        gu, act, yp = model._experts_fwd(xp, plan, P[p + "w1"], P[p + "w2"], keep)
        yr = yp[plan.dest.long()]
        back = self._exchange_nccl(yr.contiguous(), rc, sc)
        yslot = torch.empty(T * K, h2.shape[1], dtype=h2.dtype, device=h2.device)
        yslot[order] = back
        ident = torch.arange(T * K, dtype=torch.int32, device=h2.device)
        y = C.moe_combine(yslot, ident, w, T, K)
        saved = dict(plan=plan, xp=xp, gu=gu, act=act, order=order, sc=sc, rc=rc, ids=ids, w=w, probs=probs, yslot=yslot,
                     ident=ident) if keep else None
        return y, saved

    def _moe_backward_nccl(self, model, i, h2, dy, saved):
        cfg, P, G, C = self.cfg, model.store.params, model.store.grads, self.C
        p = f"layers.{i}.moe."
        ids, w, plan, order = saved["ids"], saved["w"], saved["plan"], saved["order"]
        T, K = ids.shape
        big = torch.tensor([1 << 20, 1 << 30], dtype=torch.int32, device=dy.device)
        dy_slot, dw = C.moe_combine_bwd(dy, saved["yslot"], saved["ident"], big, w)
        dyr = self._exchange_nccl(dy_slot[order].contiguous(), saved["sc"], saved["rc"])
        dyp = C.moe_permute(dyr, plan.src, plan.num_tiles, 1)
        dxp = model._experts_bwd(dyp, saved["xp"], saved["gu"], saved["act"], plan, P[p + "w1"], P[p + "w2"],
                                 G[p + "w1"], G[p + "w2"])
        back = self._exchange_nccl(dxp[plan.dest.long()].contiguous(), saved["rc"], saved["sc"])
        dslot = torch.empty_like(dy_slot)
        dslot[order] = back
        dh2 = C.moe_combine(dslot, saved["ident"], None, T, K)
        return model._router_bwd(i, h2, dh2, saved["probs"], ids, w, dw)
