"""Flat fused Adam(W) over the ``ParamStore`` buffers, with optional host-offloaded moments.

One optimizer instance covers both parameter groups of a rank: ``dense`` (replicated over ranks; its
gradient is all-reduced over the data-parallel group before the step) and ``expert`` (owned by this
rank).  Precision follows the reference's precision-aware-optimizer flags: fp32 or bf16 moments
(``--exp-avg-dtype/--exp-avg-sq-dtype``), optional fp32 master weights, and ``--optimizer-cpu-offload``
semantics for the moments — here as pinned-host chunks streamed through the GPU on side streams
(H2D of chunk i+1 and D2H of chunk i-1 overlap the update of chunk i), which is what lets a 30B-parameter
MoE train on a single 180 GB device.

Gradient clipping needs no host round trip: the squared norm is reduced on the device, the clip
coefficient and the non-finite flag stay in device memory and are consumed by the update kernel.

Reference counterparts: Megatron DistributedOptimizer + TE FusedAdam set up in
miles/backends/megatron_utils/model.py:125-210; LR schedule in samples, model.py:68-113.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist

from ..models.params import ParamStore


@dataclass
class OptimConfig:
    lr: float = 1e-6
    beta1: float = 0.9
    beta2: float = 0.98
    eps: float = 1e-8
    weight_decay: float = 0.1
    clip_grad: float = 1.0
    state_dtype: torch.dtype = torch.float32
    master_weights: bool = True           # fp32 master copy of bf16 parameters (on the GPU: bf16 weight + 16-bit remainder)
    offload_states: bool = False          # keep moments and master remainder of the expert group in pinned host memory
    offload_resident_frac: float = 0.0    # share of the offloaded moments that stays on the device after all (no stream)
    offload_chunk_elems: int = 1 << 27    # 128 Mi elements per streamed chunk
    # LR schedule (in optimizer steps)
    lr_decay_style: str = "constant"
    lr_warmup_iters: int = 0
    lr_decay_iters: int = 0
    min_lr: float = 0.0
    lr_wsd_decay_iters: int = 0
    skip_nonfinite: bool = True           # a non-finite gradient norm skips the step (--no-check-for-nan-in-loss-and-grad: apply anyway)


def lr_at(cfg: OptimConfig, step: int) -> float:
    """constant / linear / cosine / WSD schedule with linear warm-up (Megatron-compatible shapes)."""
    if cfg.lr_warmup_iters > 0 and step < cfg.lr_warmup_iters:
        return cfg.lr * (step + 1) / cfg.lr_warmup_iters
    if cfg.lr_decay_style == "constant" or cfg.lr_decay_iters <= 0:
        return cfg.lr
    t = min(max(step - cfg.lr_warmup_iters, 0) / max(cfg.lr_decay_iters - cfg.lr_warmup_iters, 1), 1.0)
    if cfg.lr_decay_style == "linear":
        coeff = 1.0 - t
    elif cfg.lr_decay_style == "cosine":
        coeff = 0.5 * (1.0 + math.cos(math.pi * t))
    elif cfg.lr_decay_style == "WSD":
        start = cfg.lr_decay_iters - cfg.lr_wsd_decay_iters
        coeff = 1.0 if step < start else max(0.0, 1.0 - (step - start) / max(cfg.lr_wsd_decay_iters, 1))
    else:
        raise ValueError(f"unknown lr_decay_style {cfg.lr_decay_style!r}")
    return cfg.min_lr + (cfg.lr - cfg.min_lr) * coeff


class FlatAdam:
    def __init__(self, store: ParamStore, cfg: OptimConfig, dp_group=None, ep_group=None, tp_group=None, dense_shard=None,
                 pp_group=None, shard_group=None):
        self.store, self.cfg = store, cfg
        self.dp_group, self.ep_group = dp_group, ep_group
        self.shard_group = shard_group  # a sharded store: every rank holds a different slice of every gradient
        self.tp_group = tp_group  # tensor-parallel shards count once each in the global gradient norm
        self.pp_group = pp_group  # pipeline stages hold disjoint layers: their squared norms add up
        self.dev = store.device
        self.on_gpu = self.dev.type == "cuda"
        self.step_count = 0
        self.C = None
        if self.on_gpu:
            from ..ops import _ext

            self.C = _ext.load(required=True)
        self.launches = 0
        self.state: dict = {}
        # replicated parameters partitioned over the data-parallel ranks (parallel/dp_optimizer.py): this rank holds
        # states for its range only and the step runs as peer-memory kernels instead of all-reduce + replicated Adam
        self.dense_shard = dense_shard
        for g, flat in store.flat.items():
            n = flat.numel()
            if n == 0:
                continue
            if g == "dense" and dense_shard is not None:
                self.state[g] = {"offload": False, "sharded": True, "m": dense_shard.m, "v": dense_shard.v,
                                 "master": dense_shard.master}
                continue
            off = cfg.offload_states and g == "expert" and self.on_gpu
            st: dict = {"offload": off}
            # split master: the bf16 weight is the upper half of the fp32 master, `lo` the signed 16-bit remainder
            # (starts at zero: the initial master is the bf16 weight itself)
            split = cfg.master_weights and flat.dtype == torch.bfloat16 and self.on_gpu
            if off:
                ce = cfg.offload_chunk_elems
                st["chunks"] = [(a, min(a + ce, n)) for a in range(0, n, ce)]
                # spread the chunks that stay on the device evenly among the streamed ones, so that their updates
                # fill the time the copy engines need for the next streamed chunk
                fr = min(max(cfg.offload_resident_frac, 0.0), 1.0)
                res = [int((i + 1) * fr) > int(i * fr) for i in range(len(st["chunks"]))]

                def mk(k, on_dev, dt=cfg.state_dtype):
                    if on_dev:
                        return torch.zeros(k, dtype=dt, device=self.dev)
                    return torch.empty(k, dtype=dt, pin_memory=True).zero_()  # pinned directly: no pageable detour

                st["m"] = [mk(b - a, r) for (a, b), r in zip(st["chunks"], res)]
                st["v"] = [mk(b - a, r) for (a, b), r in zip(st["chunks"], res)]
                st["master"] = None
                # the 16-bit remainder of the split fp32 master travels with the moments of its chunk
                st["lo"] = [mk(b - a, r, torch.int16) for (a, b), r in zip(st["chunks"], res)] if split else None
            else:
                st["m"] = torch.zeros(n, dtype=cfg.state_dtype, device=self.dev)
                st["v"] = torch.zeros(n, dtype=cfg.state_dtype, device=self.dev)
                st["lo"] = torch.zeros(n, dtype=torch.int16, device=self.dev) if split else None
                st["master"] = flat.float().clone() if (cfg.master_weights and flat.dtype != torch.float32 and not split) else None
            self.state[g] = st
        # weight decay applies to matrices only (norm weights and biases are exempt)
        self.segments = {g: [] for g in store.flat}
        custom = getattr(store, "decay_segments", None)
        if custom is not None:
            self.segments = custom(cfg.weight_decay)  # a sharded store knows which of its elements are matrices
        for s in (store.specs if custom is None else ()):
            wd = cfg.weight_decay if len(s.shape) >= 2 else 0.0
            segs = self.segments[s.group]
            if segs and segs[-1][2] == wd and segs[-1][1] == s.offset:
                segs[-1] = (segs[-1][0], s.offset + ((s.numel + 127) // 128) * 128, wd)
            else:
                segs.append((s.offset, s.offset + ((s.numel + 127) // 128) * 128, wd))
        self.norm_buf = torch.zeros(2, dtype=torch.float32, device=self.dev)  # [dense sumsq, expert sumsq]
        self.grad_scale = torch.ones(1, dtype=torch.float32, device=self.dev)
        self.skip_flag = torch.zeros(1, dtype=torch.float32, device=self.dev)
        self.last_grad_norm: Optional[torch.Tensor] = None
        self._streams = None
        self.h2d_bytes = 0
        self.d2h_bytes = 0

    # ------------------------------------------------------------------ gradient norm / clipping
    def _sumsq(self, g: torch.Tensor, out: torch.Tensor) -> None:
        if self.C is not None:
            self.C.sumsq(g, out)
            self.launches += 1
        else:
            out += g.float().pow(2).sum()

    def compute_grad_norm(self) -> torch.Tensor:
        """Global L2 norm over dense (counted once) and expert (summed over EP ranks) gradients."""
        self.norm_buf.zero_()
        for i, g in enumerate(("dense", "expert")):
            gr = self.store.grad.get(g)
            if g == "dense" and self.dense_shard is not None:
                ss = self.dense_shard.reduce().reshape(1)  # the reduce-scatter; the shards' sums of squares add up
                dist.all_reduce(ss, group=self.dp_group)
                self.norm_buf[0:1] = ss
                self.launches += 3
                continue
            if gr is not None and gr.numel():
                self._sumsq(gr, self.norm_buf[i:i + 1])
        if self.ep_group is not None and dist.is_initialized() and dist.get_world_size(self.ep_group) > 1:
            dist.all_reduce(self.norm_buf[1:2], group=self.ep_group)
        if self.tp_group is not None and dist.is_initialized() and dist.get_world_size(self.tp_group) > 1:
            # dense = replicated tensors (identical on every tensor-parallel rank, counted once) + sharded ones
            # (each rank holds a different part): sum the sharded part over the group
            from ..models.params import is_tp_sharded

            sharded = torch.zeros(1, dtype=torch.float32, device=self.dev)
            for name, g in self.store.grads.items():
                if is_tp_sharded(name):
                    sharded += g.float().pow(2).sum()
            total_sharded = sharded.clone()
            dist.all_reduce(total_sharded, group=self.tp_group)
            self.norm_buf[0:1] += total_sharded - sharded
        if self.pp_group is not None and dist.is_initialized() and dist.get_world_size(self.pp_group) > 1:
            dist.all_reduce(self.norm_buf, group=self.pp_group)
        if self.shard_group is not None and dist.is_initialized() and dist.get_world_size(self.shard_group) > 1:
            dist.all_reduce(self.norm_buf, group=self.shard_group)
        total = self.norm_buf.sum().sqrt()
        self.last_grad_norm = total
        return total

    def _prepare_scale(self, extra_scale: float) -> None:
        norm = self.compute_grad_norm()
        finite = torch.isfinite(norm)
        if self.cfg.skip_nonfinite:
            self.skip_flag.copy_((~finite).float().reshape(1))
        else:
            self.skip_flag.zero_()
        if self.cfg.clip_grad and self.cfg.clip_grad > 0:
            coef = torch.clamp(self.cfg.clip_grad / (norm * extra_scale + 1e-6), max=1.0)
        else:
            coef = torch.ones((), device=self.dev)
        self.grad_scale.copy_((coef * extra_scale).reshape(1))

    # ------------------------------------------------------------------ update
    def _adam_region(self, p, master, g, m, v, lr, wd, step, lo=None):
        c = self.cfg
        if self.C is not None and p.dtype == torch.bfloat16:
            self.C.adam_step(p, master, g, m, v, lr, c.beta1, c.beta2, c.eps, wd, step, self.grad_scale, self.skip_flag, lo)
            self.launches += 1
            return
        if float(self.skip_flag.item()) != 0.0:
            return
        grad = g.float() * self.grad_scale
        w = master if master is not None else p.float()
        mf, vf = m.float(), v.float()
        mf.mul_(c.beta1).add_(grad, alpha=1 - c.beta1)
        vf.mul_(c.beta2).addcmul_(grad, grad, value=1 - c.beta2)
        upd = (mf / (1 - c.beta1 ** step)) / ((vf / (1 - c.beta2 ** step)).sqrt() + c.eps)
        w = w - lr * (upd + wd * w)
        m.copy_(mf)
        v.copy_(vf)
        if master is not None:
            master.copy_(w)
        p.copy_(w)

    def step(self, grad_scale: float = 1.0) -> torch.Tensor:
        """Clip, update every group, advance the schedule. ``grad_scale`` is folded into the gradients
        (e.g. 1/global_batch when the loss was accumulated un-normalised). Returns the pre-clip grad norm."""
        self.step_count += 1
        lr = lr_at(self.cfg, self.step_count - 1)
        self._prepare_scale(grad_scale)
        for g, st in self.state.items():
            flat, grad = self.store.flat[g], self.store.grad[g]
            if st["offload"]:
                self._step_offloaded(g, st, flat, grad, lr)
                continue
            if st.get("sharded"):
                self.dense_shard.apply(self.segments[g], lr, self.step_count, self.grad_scale, self.skip_flag)
                self.launches += len(self.segments[g]) + 2
                continue
            for a, b, wd in self.segments[g]:
                b = min(b, flat.numel())
                self._adam_region(flat[a:b], st["master"][a:b] if st["master"] is not None else None, grad[a:b],
                                  st["m"][a:b], st["v"][a:b], lr, wd, self.step_count,
                                  st["lo"][a:b] if st.get("lo") is not None else None)
        self.store.version += 1
        return self.last_grad_norm * grad_scale

    def _step_offloaded(self, g, st, flat, grad, lr):
        """Stream pinned-host moments through three rotating device staging buffers."""
        c = self.cfg
        if self._streams is None:
            self._streams = (torch.cuda.Stream(), torch.cuda.Stream())
        s_in, s_out = self._streams
        main = torch.cuda.current_stream()
        ce = max(b - a for a, b in st["chunks"])
        nbuf = 3
        has_lo = st.get("lo") is not None
        if "stage" not in st:
            st["stage"] = [(torch.empty(ce, dtype=c.state_dtype, device=self.dev), torch.empty(ce, dtype=c.state_dtype, device=self.dev),
                            torch.empty(ce, dtype=torch.int16, device=self.dev) if has_lo else None)
                           for _ in range(nbuf)]
        ev_in = [torch.cuda.Event() for _ in st["chunks"]]
        ev_cmp = [torch.cuda.Event() for _ in st["chunks"]]
        ev_out = [torch.cuda.Event() for _ in st["chunks"]]
        wd = self.cfg.weight_decay
        start = torch.cuda.Event()
        start.record(main)
        es = torch.empty((), dtype=c.state_dtype).element_size()
        streamed = [k for k, t in enumerate(st["m"]) if not t.is_cuda]
        order = {k: j for j, k in enumerate(streamed)}
        for k, (a, b) in enumerate(st["chunks"]):
            if st["m"][k].is_cuda:  # resident chunk: plain update, overlaps the copies of the streamed ones
                self._adam_region(flat[a:b], None, grad[a:b], st["m"][k], st["v"][k], lr, wd, self.step_count,
                                  st["lo"][k] if has_lo else None)
                continue
            i = order[k]
            dm, dv, dl = st["stage"][i % nbuf]
            n = b - a
            with torch.cuda.stream(s_in):
                if i >= nbuf:
                    s_in.wait_event(ev_out[i - nbuf])  # staging buffer drained
                else:
                    s_in.wait_event(start)
                dm[:n].copy_(st["m"][k], non_blocking=True)
                dv[:n].copy_(st["v"][k], non_blocking=True)
                if has_lo:
                    dl[:n].copy_(st["lo"][k], non_blocking=True)
                ev_in[i].record(s_in)
            main.wait_event(ev_in[i])
            self._adam_region(flat[a:b], None, grad[a:b], dm[:n], dv[:n], lr, wd, self.step_count, dl[:n] if has_lo else None)
            ev_cmp[i].record(main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_cmp[i])
                st["m"][k].copy_(dm[:n], non_blocking=True)
                st["v"][k].copy_(dv[:n], non_blocking=True)
                if has_lo:
                    st["lo"][k].copy_(dl[:n], non_blocking=True)
                ev_out[i].record(s_out)
            self.h2d_bytes += n * (2 * es + (2 if has_lo else 0))
            self.d2h_bytes += n * (2 * es + (2 if has_lo else 0))
        if streamed:
            main.wait_event(ev_out[len(streamed) - 1])
            if len(streamed) > 1:
                main.wait_event(ev_out[len(streamed) - 2])

    def promote_offloaded(self, max_bytes: int) -> int:
        """Move evenly spaced chunks of the host-resident moments to the device, up to ``max_bytes``. Called once
        everything else (engine, KV cache, exchange buffers) is allocated, with what is then really free minus the
        activation reserve: the streamed volume shrinks by what fits. Returns the bytes moved."""
        moved = 0
        for st in self.state.values():
            if not st.get("offload"):
                continue
            host = [k for k, t in enumerate(st["m"]) if not t.is_cuda]
            if not host:
                continue
            per = st["m"][host[0]].numel() * (2 * st["m"][host[0]].element_size() + (2 if st.get("lo") is not None else 0))
            take = min(len(host), int(max(max_bytes - moved, 0) // max(per, 1)))
            if take <= 0:
                continue
            stride = len(host) / take
            for j in range(take):
                k = host[min(len(host) - 1, int(j * stride))]
                if st["m"][k].is_cuda:
                    continue
                st["m"][k] = st["m"][k].to(self.dev)
                st["v"][k] = st["v"][k].to(self.dev)
                if st.get("lo") is not None:
                    st["lo"][k] = st["lo"][k].to(self.dev)
                moved += per
        return moved

    # ------------------------------------------------------------------ checkpoint
    def state_dict(self) -> dict:
        out = {"step": self.step_count}
        for g, st in self.state.items():
            if st["offload"]:
                out[g] = {"m": torch.cat([t.cpu() for t in st["m"]]), "v": torch.cat([t.cpu() for t in st["v"]]), "master": None,
                          "lo": torch.cat([t.cpu() for t in st["lo"]]) if st.get("lo") is not None else None}
            else:
                out[g] = {"m": st["m"], "v": st["v"], "master": st["master"], "lo": st.get("lo")}
        return out

    def master_fp32(self, g: str) -> torch.Tensor:
        """The fp32 master values of group ``g`` as one tensor (a copy; for checkpoints, exports and checks)."""
        st, flat = self.state[g], self.store.flat[g]
        if st.get("sharded"):
            return flat.float()
        if st.get("master") is not None:
            return st["master"].clone()
        lo = st.get("lo")
        if lo is None:
            return flat.float()
        if isinstance(lo, list):
            out = torch.empty(flat.numel(), dtype=torch.float32, device=self.dev)
            for (a, b), l in zip(st["chunks"], lo):
                out[a:b] = self.C.split_master_join(flat[a:b], l.to(self.dev, non_blocking=True))
            return out
        return self.C.split_master_join(flat, lo)

    def load_state_dict(self, sd: dict) -> None:
        self.step_count = int(sd.get("step", 0))
        for g, st in self.state.items():
            if g not in sd:
                continue
            src = sd[g]
            if st["offload"]:
                for k, ((a, b), m, v) in enumerate(zip(st["chunks"], st["m"], st["v"])):
                    m.copy_(src["m"][a:b])
                    v.copy_(src["v"][a:b])
                    if st.get("lo") is not None:
                        if src.get("lo") is not None:
                            st["lo"][k].copy_(src["lo"][a:b])
                        else:
                            st["lo"][k].zero_()
            else:
                st["m"].copy_(src["m"])
                st["v"].copy_(src["v"])
                if st["master"] is not None and src.get("master") is not None:
                    st["master"].copy_(src["master"])
                if st.get("lo") is not None:
                    if src.get("lo") is not None:
                        st["lo"].copy_(src["lo"])
                    elif src.get("master") is not None:  # a checkpoint written with a plain fp32 master
                        self.C.split_master_cut(src["master"].to(self.dev).float().contiguous(), self.store.flat[g], st["lo"])
                    else:
                        st["lo"].zero_()

    def reset_state(self) -> None:
        for st in self.state.values():
            for key in ("m", "v"):
                ts = st[key] if isinstance(st[key], list) else [st[key]]
                for t in ts:
                    t.zero_()
        self.step_count = 0

    def sync_master_from_params(self) -> None:
        for g, st in self.state.items():
            if st.get("sharded"):
                self.dense_shard.sync_master_from_params()
            elif st.get("master") is not None:
                st["master"].copy_(self.store.flat[g].float())
            elif st.get("lo") is not None:  # the master becomes the bf16 weight itself: remainder zero
                for t in (st["lo"] if isinstance(st["lo"], list) else [st["lo"]]):
                    t.zero_()
