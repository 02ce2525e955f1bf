"""Expert-parallel MoE for decode steps: the low-latency exchange of ``csrc/ep_decode.cu`` around the grouped
expert GEMMs.

The rollout engine of an expert-parallel trainer keeps every rank's own sequences on that rank (attention and
the dense projections are data parallel) and serves the experts where they live, so the expert weights, the bulk
of what a decode step streams from HBM, are read once per *group* instead of once per GPU. Per MoE layer and
decode step a rank launches::

    router GEMV -> send (norm + top-k + row / id stores to the owners, flags)
                -> plan (wait for all sources, sort local picks by expert)
                -> permute -> grouped GEMM -> SwiGLU -> grouped GEMM
                -> return (gate-weighted partial sums stored at the sources, flags)
                -> combine (wait for all owners, add partial sums to the residual)

All of it is captured in the engine's decode CUDA graph: the epochs the flags carry live in device memory. Every
rank must run the same number of decode steps with the same row bound (the engine agrees on both, see
``engine/core.py``); rows a rank pads its batch with are announced as "no expert" and cost no expert work.

Reference: the reference serves this model with expert-parallel SGLang engines and DeepEP's low-latency
dispatch (scripts/run_qwen3_30b_a3b.py:311-358).
"""
from __future__ import annotations

import torch

from ..ops import _ext
from .symm import SymmetricRegion


class EpDecodeLL:
    low_latency = True

    def __init__(self, cfg, ps, max_rows: int = 64, wait_ms: float = 1000.0):
        assert ps.device.type == "cuda", "the low-latency exchange runs on CUDA devices"
        self.cfg, self.ps = cfg, ps
        self.group, self.rank, self.n = ps.ep.group, ps.ep.rank, ps.ep.size
        assert cfg.num_experts % self.n == 0
        self.el = cfg.num_experts // self.n
        self.E, self.K, self.H = cfg.num_experts, cfg.moe_top_k, cfg.hidden_size
        self.Bm = int(max_rows)
        self.dev = ps.device
        self.C = _ext.load(required=True)
        self.wait_ns = int(wait_ms * 1e6)
        R, Bm, H, K = self.n, self.Bm, self.H, self.K

        def al(x):
            return (x + 255) // 256 * 256

        off, sizes = 0, {}
        for name, nb in (("xg", R * Bm * H * 2), ("ig", R * Bm * K * 4), ("wg", R * Bm * K * 4), ("yb", R * Bm * H * 2),
                         ("flag_a", R * 8), ("flag_b", R * 8)):
            sizes[name] = off
            off = al(off + nb)
        self.region = SymmetricRegion(off, self.group, self.rank, R, self.dev)
        self.bases = list(self.region.peer_base)
        self.layout = [R, Bm, H, K, sizes["xg"], sizes["ig"], sizes["wg"], sizes["yb"], sizes["flag_a"], sizes["flag_b"]]
        self.xg = self.C.tensor_from_ptr(self.region.base + sizes["xg"], [R * Bm, H], torch.bfloat16, self.dev.index or 0)
        self.ctrl = torch.zeros(8, dtype=torch.int64, device=self.dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.dev)
        self.rows = Bm        # row bound of the current step (every rank uses the same one)
        self.active = None    # int32 [rows] of the current step: 0 marks a padding row
        self.bytes_sent = 0

    def set_step(self, rows: int, active) -> None:
        """Row bound (identical on every rank) and padding mask for the decode steps that follow."""
        assert 1 <= rows <= self.Bm
        self.rows, self.active = int(rows), active

    def check_status(self) -> None:
        code = int(self.status.item())
        if code:
            self.status.zero_()
            raise RuntimeError(f"expert-parallel decode exchange reported error {code} "
                               "(5 = a source rank's rows never arrived, 6 = an owner rank's results never arrived)")

    def moe_decode(self, model, i: int, x2: torch.Tensor, h2, record=None) -> torch.Tensor:
        """``x2 + MoE(RMSNorm(x2))`` for the rows of this rank. ``h2``: the normalised rows if the caller already has
        them (more than eight rows), else None and the norm is folded into the router GEMV and the send kernel."""
        cfg, P, C = self.cfg, model.store.params, self.C
        p = f"layers.{i}."
        T = x2.shape[0]
        assert T <= self.rows, f"{T} rows exceed the agreed row bound {self.rows}"
        ln2 = P[p + "ln2.weight"]
        if h2 is None:
            logits = torch.empty(T, self.E, dtype=torch.float32, device=x2.device)
            C.small_gemv(x2, ln2, cfg.rms_eps, P[p + "moe.router.weight"], None, logits, model.status)
            rows_in, ln = x2, ln2
        else:
            logits = model.linear(h2, P[p + "moe.router.weight"], torch.float32)
            rows_in, ln = h2, None
        ids = torch.empty(T, self.K, dtype=torch.int32, device=x2.device)
        w = torch.empty(T, self.K, dtype=torch.float32, device=x2.device)
        active = self.active[:T] if self.active is not None else None
        C.ep_ll_send(rows_in, ln, cfg.rms_eps, logits, active, self.bases, self.layout, self.rank, cfg.norm_topk_prob, ids, w,
                     self.ctrl)
        if record is not None:
            record.append(ids)
        src_rows, counts, offsets, dest, row_src, tiles, totals = C.ep_ll_plan(
            self.region.base, self.layout, self.rank, self.E, self.rows, 1, self.ctrl, self.wait_ns, self.status)
        from ..models.b200_impl import MoeCtx

        plan = MoeCtx(None, None, None, offsets, dest, row_src, tiles, totals, row_src.numel())
        xp = C.moe_permute(self.xg, row_src, totals, self.K)
        _, _, yp = model._experts_fwd(xp, plan, P[p + "moe.w1"], P[p + "moe.w2"], keep=False)
        C.ep_ll_return(yp, dest, src_rows, self.bases, self.layout, self.rank, self.rows, self.ctrl)
        y = C.ep_ll_combine(self.region.base, self.layout, ids, active, x2, self.E, self.ctrl, self.wait_ns, self.status)
        model.launches += 6
        self.bytes_sent += T * self.H * 2 * (self.n - 1)
        return y
