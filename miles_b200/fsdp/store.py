"""Sharded parameter store: the same interface as ``models.params.ParamStore``, one ``1 / shard_size`` slice of every
unit per rank.

Layout. The parameters keep the order and the 128-element alignment of ``build_specs``; a *unit* (``embed``,
``layers.i``, ``head``) is a contiguous range of the ``dense`` flat buffer and one of the ``expert`` flat buffer. Each
range is padded to a multiple of ``shard_size * 128`` elements and cut into ``shard_size`` equal pieces; rank ``r`` keeps
piece ``r`` of every unit, back to back, in ``flat[group]`` (so the optimizer, the weight back-ups and the per-rank
checkpoint code see one flat buffer per group, as with the unsharded store). ``grad[group]`` is the fp32 gradient of
that buffer.

Materialisation. ``params[name]`` returns a view into a buffer that holds the whole unit of ``name``:

* without autograd (the hand-written forward / backward, and every no-grad forward) a unit is all-gathered into one of
  ``num_buffers`` rotating buffers on a communication stream; looking up a unit also starts the gather of its neighbour
  in the direction the model is walking (forward: next layer, backward: previous layer), which then overlaps the
  current unit's kernels; the gather into a recycled buffer is ordered behind everything already queued on the compute
  stream, so kernels still reading the old unit finish first. ``grads[name]`` is a view into a zeroed full-unit gradient
  buffer; when the backward moves on to another unit the buffer is reduce-scattered and added into ``grad[group]``
  (``finish_grads`` flushes the last one).
* under autograd (``on_requires_grad(True)``) the gather is an autograd function whose backward is the
  reduce-scatter, and the shard buffers are the leaves.

Everything here is collective over the shard group: all its ranks must look up the same units in the same order
(the trainer equalises micro-batch counts across ranks for that reason).

Reference behaviour: ``fully_shard`` per decoder layer + root with bf16 parameters and fp32 reduction
(miles/backends/fsdp_utils/actor.py:717-761).
"""
from __future__ import annotations

import contextlib
from collections import OrderedDict
from collections.abc import Mapping
from dataclasses import dataclass, field
from typing import Iterator, Optional

import torch
import torch.distributed as dist

from ..models.config import ModelConfig
from ..models.params import ParamStore, build_specs

ALIGN = 128


def unit_key(name: str) -> str:
    if name.startswith("layers."):
        return "layers." + name.split(".")[1]
    return "embed" if name == "embed.weight" else "head"


@dataclass
class Unit:
    index: int
    name: str
    specs: list = field(default_factory=list)
    lo: dict = field(default_factory=dict)       # group -> first element in the full flat buffer
    hi: dict = field(default_factory=dict)       # group -> end (exclusive, aligned)
    padded: dict = field(default_factory=dict)   # group -> padded length (multiple of shard_size * 128; 0 = none)
    shard_off: dict = field(default_factory=dict)  # group -> where this unit's piece starts in the rank's flat buffer

    def piece(self, g: str, shard_size: int) -> int:
        return self.padded[g] // shard_size


def build_units(specs: list, shard_size: int) -> list:
    units: "OrderedDict[str, Unit]" = OrderedDict()
    for s in specs:
        k = unit_key(s.name)
        u = units.get(k)
        if u is None:
            u = units[k] = Unit(len(units), k)
        u.specs.append(s)
        end = s.offset + (s.numel + ALIGN - 1) // ALIGN * ALIGN
        u.lo[s.group] = min(u.lo.get(s.group, s.offset), s.offset)
        u.hi[s.group] = max(u.hi.get(s.group, end), end)
    off = {"dense": 0, "expert": 0}
    q = shard_size * ALIGN
    out = list(units.values())
    for u in out:
        for g in ("dense", "expert"):
            n = u.hi.get(g, 0) - u.lo.get(g, 0)
            u.lo.setdefault(g, 0)
            u.hi.setdefault(g, 0)
            u.padded[g] = (n + q - 1) // q * q
            u.shard_off[g] = off[g]
            off[g] += u.padded[g] // shard_size
    return out


def _all_gather(out: torch.Tensor, piece: torch.Tensor, group, size: int) -> None:
    if size == 1:
        out.copy_(piece)
        return
    piece = piece.contiguous()
    if piece.dtype in (torch.int16, torch.uint16):
        # a gather only moves bytes, and not every backend knows 16-bit integers (the remainder words of the split
        # fp32 master weights): send them as bytes
        out, piece = out.view(torch.uint8), piece.view(torch.uint8)
    dist.all_gather_into_tensor(out, piece, group=group)


def _reduce_scatter(out: torch.Tensor, full: torch.Tensor, group, size: int) -> None:
    if size == 1:
        out.copy_(full)
    else:
        dist.reduce_scatter_tensor(out, full.contiguous(), op=dist.ReduceOp.SUM, group=group)


class _GatherUnit(torch.autograd.Function):
    """All-gather of one unit's pieces; the backward reduce-scatters the unit's gradient onto the pieces."""

    @staticmethod
    def forward(ctx, piece: torch.Tensor, group, size: int):
        ctx.group, ctx.size = group, size
        out = piece.new_empty(piece.numel() * size)
        _all_gather(out, piece.detach(), group, size)
        return out

    @staticmethod
    def backward(ctx, g: torch.Tensor):
        out = g.new_empty(g.numel() // ctx.size)
        _reduce_scatter(out, g, ctx.group, ctx.size)
        return out, None, None


class _Lazy(Mapping):
    def __init__(self, store: "FsdpParamStore", getter, active):
        self._s, self._get, self._active = store, getter, active

    def __getitem__(self, name: str) -> torch.Tensor:
        if name not in self._s.by_name:
            raise KeyError(name)
        return self._get(name)

    def __contains__(self, name) -> bool:
        return name in self._s.by_name

    def __iter__(self):
        return iter(self._s.by_name)

    def __len__(self) -> int:
        return len(self._s.by_name) if self._active() else 0

    def __setitem__(self, name, value) -> None:
        pass  # views are made on demand: callers that "rebuild" them have nothing to store

    def clear(self) -> None:
        pass


class _Slot:
    __slots__ = ("buffer", "views", "ready", "waited")

    def __init__(self, buffer: int, views: dict, ready):
        self.buffer, self.views, self.ready, self.waited = buffer, views, ready, ready is None


class FsdpParamStore:
    is_fsdp = True

    def __init__(self, cfg: ModelConfig, device, dtype: torch.dtype, mesh, init_std: float = 0.02, seed: int = 1234,
                 init: bool = True, num_buffers: int = 2, prefetch: bool = True):
        self.cfg = self.global_cfg = cfg
        self.tp_size, self.tp_rank, self.ep_size, self.ep_rank, self.pp_size, self.pp_rank = 1, 0, 1, 0, 1, 0
        self.layer_range = (0, cfg.num_layers)
        self.is_first_stage = self.is_last_stage = True
        self.device = torch.device(device)
        self.dtype = dtype
        self.mesh = mesh
        self.shard_size, self.shard_rank, self.group = mesh.shard.size, mesh.shard.rank, mesh.shard.group
        self.specs = build_specs(cfg)
        self.by_name = OrderedDict((s.name, s) for s in self.specs)
        self.units = build_units(self.specs, self.shard_size)
        self.unit_of = {s.name: u for u in self.units for s in u.specs}
        self.full_sizes = {g: max((u.hi[g] for u in self.units), default=0) for g in ("dense", "expert")}
        self.sizes = {g: sum(u.piece(g, self.shard_size) for u in self.units) for g in ("dense", "expert")}
        self.max_padded = {g: max((u.padded[g] for u in self.units), default=0) for g in ("dense", "expert")}
        self.flat = {g: torch.zeros(n, dtype=dtype, device=self.device) for g, n in self.sizes.items()}
        self.grad: dict = {"dense": None, "expert": None}
        self.params = _Lazy(self, self._param, lambda: True)
        self.grads = _Lazy(self, self._grad_view, lambda: self.grad["dense"] is not None)
        self.version = 0
        self.num_buffers, self.prefetch = max(1, num_buffers), prefetch and num_buffers >= 2
        self._pbuf: list = []            # parameter buffers: [{group: tensor}] * num_buffers
        self._free: list = []
        self._live: "OrderedDict[int, _Slot]" = OrderedDict()
        self._last: Optional[int] = None
        self._dir = 1
        self._comm = torch.cuda.Stream(self.device) if self.device.type == "cuda" else None
        self._gdt = {"dense": torch.float32, "expert": torch.float32}
        self._gbuf: list = []            # full-unit gradient buffers (two, used in turn)
        self._gdone: list = []           # per gradient buffer: event of the reduce-scatter that last read it
        self._gnext = 0
        self._gcur = None                # (unit, buffer index, views)
        self._rs_tmp: dict = {}
        self._autograd = False
        self._ag_live: "OrderedDict[int, dict]" = OrderedDict()
        self._write = None               # (gather_first,) while inside writing()
        self._wcur: Optional[Unit] = None
        self.gathers = 0                 # collectives issued (all-gathers / reduce-scatters), for tests and profiles
        self.reduce_scatters = 0
        if init:
            self.init_weights(init_std, seed)

    # ------------------------------------------------------------------ construction
    @torch.no_grad()
    def init_weights(self, std: float = 0.02, seed: int = 1234) -> None:
        """The same values as the unsharded store draws for this seed (every value is a function of seed, parameter
        name and element index), unit by unit, each rank keeping its piece."""
        with self.writing(gather=False):
            ParamStore.init_weights(self, std, seed)

    # ------------------------------------------------------------------ buffers
    def _param_buffers(self) -> None:
        if not self._pbuf:
            self._pbuf = [{g: torch.empty(n, dtype=self.dtype, device=self.device) for g, n in self.max_padded.items()}
                          for _ in range(self.num_buffers)]
            self._free = list(range(self.num_buffers))

    def release_buffers(self) -> None:
        """Drop the unit buffers (parameters and gradients); they come back on the next use."""
        self.invalidate()
        self._pbuf, self._free, self._gbuf, self._gdone, self._rs_tmp = [], [], [], [], {}

    def invalidate(self) -> None:
        """Forget every materialised unit (the shards changed, or a new pass starts)."""
        if self._comm is not None and self._live:
            torch.cuda.current_stream(self.device).wait_stream(self._comm)
        self._live.clear()
        self._ag_live.clear()
        self._free = list(range(len(self._pbuf)))
        self._last, self._dir = None, 1

    def begin_pass(self) -> None:
        """Called by the model at the start of every forward: units are never carried from one pass to the next
        (the weights may have been stepped or swapped in between)."""
        self.invalidate()

    def _views(self, u: Unit, bufs: dict) -> dict:
        return {s.name: bufs[s.group][s.offset - u.lo[s.group]:s.offset - u.lo[s.group] + s.numel].view(s.shape) for s in u.specs}

    def _piece(self, flat: torch.Tensor, u: Unit, g: str) -> torch.Tensor:
        n = u.piece(g, self.shard_size)
        return flat[u.shard_off[g]:u.shard_off[g] + n]

    def _gather_now(self, u: Unit, bufs: dict, flats: Optional[dict] = None) -> None:
        """All-gather unit ``u`` of ``flats`` (default: the weights) into ``bufs`` on the current stream."""
        flats = flats if flats is not None else self.flat
        for g in ("dense", "expert"):
            if u.padded[g] and flats.get(g) is not None:
                _all_gather(bufs[g][:u.padded[g]], self._piece(flats[g], u, g), self.group, self.shard_size)
                self.gathers += 1

    def _take_buffer(self, keep: Optional[int]) -> int:
        if self._free:
            return self._free.pop()
        for idx in self._live:
            if idx != keep:
                return self._live.pop(idx).buffer
        raise RuntimeError("no unit buffer free: num_buffers is too small for this access pattern")

    def _ensure(self, u: Unit, keep: Optional[int] = None) -> _Slot:
        slot = self._live.get(u.index)
        if slot is not None:
            return slot
        self._param_buffers()
        b = self._take_buffer(keep if keep is not None else u.index)
        bufs = self._pbuf[b]
        ready = None
        if self._comm is not None:
            # behind everything queued so far on the compute stream: kernels still reading the unit this buffer held,
            # and whatever last wrote the shards
            self._comm.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(self._comm):
                self._gather_now(u, bufs)
                ready = torch.cuda.Event()
                ready.record(self._comm)
        else:
            self._gather_now(u, bufs)
        slot = _Slot(b, self._views(u, bufs), ready)
        self._live[u.index] = slot
        return slot

    # ------------------------------------------------------------------ parameter lookup
    def _param(self, name: str) -> torch.Tensor:
        u = self.unit_of[name]
        if self._write is not None:
            return self._write_view(u, name)
        if self._autograd and torch.is_grad_enabled():
            return self._autograd_view(u, name)
        slot = self._ensure(u)
        if not slot.waited:
            torch.cuda.current_stream(self.device).wait_event(slot.ready)
            slot.waited = True
        self._live.move_to_end(u.index)
        if u.index != self._last:
            if self._last is not None:
                self._dir = 1 if u.index > self._last else -1
            self._last = u.index
            nxt = u.index + self._dir
            if self.prefetch and 0 <= nxt < len(self.units) and nxt not in self._live:
                self._ensure(self.units[nxt], keep=u.index)
        return slot.views[name]

    def _autograd_view(self, u: Unit, name: str) -> torch.Tensor:
        views = self._ag_live.get(u.index)
        if views is None:
            fulls = {g: _GatherUnit.apply(self._piece(self.flat[g], u, g), self.group, self.shard_size)
                     for g in ("dense", "expert") if u.padded[g]}
            self.gathers += len(fulls)
            views = self._views(u, fulls)
            self._ag_live[u.index] = views
            while len(self._ag_live) > 2:
                self._ag_live.popitem(last=False)  # autograd keeps what the backward still needs
        return views[name]

    def on_requires_grad(self, flag: bool) -> None:
        """The autograd model path turns gradient tracking of the leaves (the shard buffers) on and off around a step."""
        self._autograd = bool(flag)
        for t in self.flat.values():
            t.requires_grad_(bool(flag))
        self.invalidate()

    def __getitem__(self, name: str) -> torch.Tensor:
        return self.params[name]

    def named_parameters(self) -> Iterator[tuple]:
        """Full tensors in parameter order, one unit materialised at a time (collective). The views are valid until the
        iteration moves two units on; inside ``writing()`` what the caller writes into them is kept."""
        for s in self.specs:
            yield s.name, self.params[s.name]

    def lm_head(self) -> torch.Tensor:
        return self.params["embed.weight"] if self.cfg.tie_embeddings else self.params["lm_head.weight"]

    # ------------------------------------------------------------------ writing whole parameters
    @contextlib.contextmanager
    def writing(self, gather: bool = True):
        """Inside this context ``params[name]`` views are writable: when the caller moves on to another unit (and at the
        end) every rank copies its piece of the unit back into its shard. All ranks must write the same values
        (a checkpoint every rank reads, the seeded initialisation). ``gather=False`` skips fetching the current values
        for callers that overwrite every parameter."""
        self.invalidate()
        self._param_buffers()
        self._write, self._wcur = (gather,), None
        try:
            yield self
        finally:
            self._flush_write()
            self._write, self._wcur = None, None
            self.invalidate()

    def _write_view(self, u: Unit, name: str) -> torch.Tensor:
        bufs = self._pbuf[0]
        if self._wcur is not u:
            self._flush_write()
            if self._write[0]:
                self._gather_now(u, bufs)
            else:
                for g in ("dense", "expert"):
                    if u.padded[g]:
                        bufs[g][:u.padded[g]].zero_()
            self._wcur = u
            self._wviews = self._views(u, bufs)
        return self._wviews[name]

    @torch.no_grad()
    def _flush_write(self) -> None:
        u = self._wcur
        if u is None:
            return
        for g in ("dense", "expert"):
            n = u.piece(g, self.shard_size)
            if n:
                self._piece(self.flat[g], u, g).copy_(self._pbuf[0][g][self.shard_rank * n:(self.shard_rank + 1) * n])
        self._wcur = None

    # ------------------------------------------------------------------ gradients
    def allocate_grads(self, dtype: torch.dtype = torch.float32, expert_dtype: Optional[torch.dtype] = None,
                       expert_storage: Optional[torch.Tensor] = None) -> None:
        """fp32 gradient shards; ``dtype`` / ``expert_dtype`` are the types of the full-unit buffers the backward writes
        into (and of the reduce-scatter)."""
        self._gdt = {"dense": dtype, "expert": expert_dtype or dtype}
        for g, n in self.sizes.items():
            if self.grad[g] is None:
                self.grad[g] = torch.zeros(n, dtype=torch.float32, device=self.device)

    def _grad_buffers(self) -> None:
        if not self._gbuf:
            self._gbuf = [{g: torch.empty(n, dtype=self._gdt[g], device=self.device) for g, n in self.max_padded.items()}
                          for _ in range(2)]
            self._gdone = [None, None]
            self._rs_tmp = {g: torch.empty(n // self.shard_size, dtype=self._gdt[g], device=self.device)
                            for g, n in self.max_padded.items()}

    def _grad_view(self, name: str) -> torch.Tensor:
        assert self.grad["dense"] is not None, "allocate_grads() must be called before training"
        u = self.unit_of[name]
        if self._gcur is not None and self._gcur[0] is not u:
            self._finish_grad_unit()
        if self._gcur is None:
            self._grad_buffers()
            b = self._gnext
            self._gnext ^= 1
            if self._gdone[b] is not None:
                torch.cuda.current_stream(self.device).wait_event(self._gdone[b])
            bufs = self._gbuf[b]
            for g in ("dense", "expert"):
                if u.padded[g]:
                    bufs[g][:u.padded[g]].zero_()
            self._gcur = (u, b, self._views(u, bufs))
        return self._gcur[2][name]

    @torch.no_grad()
    def _finish_grad_unit(self) -> None:
        u, b, _ = self._gcur
        self._gcur = None
        bufs = self._gbuf[b]

        def run():
            for g in ("dense", "expert"):
                n = u.piece(g, self.shard_size)
                if not n:
                    continue
                tmp = self._rs_tmp[g][:n]
                _reduce_scatter(tmp, bufs[g][:u.padded[g]], self.group, self.shard_size)
                self.reduce_scatters += 1
                self._piece(self.grad[g], u, g).add_(tmp)

        if self._comm is not None:
            self._comm.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(self._comm):
                run()
                ev = torch.cuda.Event()
                ev.record(self._comm)
                self._gdone[b] = ev
        else:
            run()

    def finish_grads(self) -> None:
        """Flush the unit the backward ended in and make the compute stream wait for all outstanding reductions; then
        sum over the replicas of a hybrid mesh."""
        if self._gcur is not None:
            self._finish_grad_unit()
        if self._comm is not None:
            torch.cuda.current_stream(self.device).wait_stream(self._comm)
        rep = self.mesh.replicate
        if rep.size > 1:
            for g in self.grad.values():
                if g is not None and g.numel():
                    dist.all_reduce(g, group=rep.group)

    def zero_grads(self) -> None:
        self._gcur = None
        for g in self.grad.values():
            if g is not None:
                g.zero_()

    def free_grads(self) -> None:
        self.grad = {"dense": None, "expert": None}
        self._gcur = None
        self.release_buffers()

    # ------------------------------------------------------------------ optimizer support
    def decay_segments(self, weight_decay: float) -> dict:
        """``{group: [(start, end, weight decay)]}`` over this rank's flat buffers: matrices decay, norm weights and
        biases do not; padding belongs to no segment."""
        out = {g: [] for g in self.flat}
        for u in self.units:
            for s in u.specs:
                g = s.group
                n = u.piece(g, self.shard_size)
                a = s.offset - u.lo[g]
                b = a + (s.numel + ALIGN - 1) // ALIGN * ALIGN
                lo, hi = max(a, self.shard_rank * n), min(b, (self.shard_rank + 1) * n)
                if lo >= hi:
                    continue
                wd = weight_decay if len(s.shape) >= 2 else 0.0
                seg = (u.shard_off[g] + lo - self.shard_rank * n, u.shard_off[g] + hi - self.shard_rank * n, wd)
                segs = out[g]
                if segs and segs[-1][2] == wd and segs[-1][1] == seg[0]:
                    segs[-1] = (segs[-1][0], seg[1], wd)
                else:
                    segs.append(seg)
        return out

    # ------------------------------------------------------------------ whole-model transfers
    @torch.no_grad()
    def gather_into(self, dst: ParamStore) -> int:
        """All-gather every unit into the flat buffers of an unsharded store of the same model (the rollout engine's).
        Returns the bytes written."""
        assert all(dst.sizes[g] == self.full_sizes[g] for g in self.full_sizes), "destination holds another model"
        self.invalidate()
        self._param_buffers()
        moved = 0
        for u in self.units:
            for g in ("dense", "expert"):
                n = u.hi[g] - u.lo[g]
                if not n:
                    continue
                target = dst.flat[g][u.lo[g]:u.hi[g]]
                piece = self._piece(self.flat[g], u, g)
                if n == u.padded[g] and target.dtype == piece.dtype:
                    _all_gather(target, piece, self.group, self.shard_size)  # no padding: straight into place
                else:
                    buf = self._pbuf[0][g][:u.padded[g]]
                    _all_gather(buf, piece, self.group, self.shard_size)
                    target.copy_(buf[:n])
                self.gathers += 1
                moved += n * target.element_size()
        dst.version = self.version
        return moved

    @torch.no_grad()
    def scatter_from(self, src: ParamStore) -> None:
        """Take this rank's pieces out of an unsharded store that holds the same model on this rank."""
        for u in self.units:
            for g in ("dense", "expert"):
                n = u.piece(g, self.shard_size)
                if not n:
                    continue
                a = u.lo[g] + self.shard_rank * n
                b = min(a + n, u.hi[g])
                piece = self._piece(self.flat[g], u, g)
                piece.zero_()
                if b > a:
                    piece[:b - a].copy_(src.flat[g][a:b])
        self.version = src.version
        self.invalidate()

    def full_units(self, flats: dict) -> Iterator[tuple]:
        """Collective iteration over ``(unit, {group: full padded tensor})`` of any buffers laid out like the shards
        (weights, moments, master weights). The tensors are reused by the next iteration."""
        bufs: dict = {}
        for u in self.units:
            out = {}
            for g in ("dense", "expert"):
                f = flats.get(g)
                if f is None or not u.padded[g]:
                    continue
                if g not in bufs or bufs[g].dtype != f.dtype:
                    bufs[g] = torch.empty(self.max_padded[g], dtype=f.dtype, device=self.device)
                # state kept in host memory travels through the device: the group's backend moves device tensors
                _all_gather(bufs[g][:u.padded[g]], self._piece(f, u, g).to(self.device), self.group, self.shard_size)
                out[g] = bufs[g][:u.padded[g]]
            yield u, out

    # ------------------------------------------------------------------ bookkeeping
    def num_local_params(self) -> int:
        return sum(self.sizes.values())

    def num_global_params(self) -> int:
        return sum(s.numel for s in self.specs)

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.flat.values())

    def checksum(self) -> dict:
        """Per-group sums of absolute values over the whole model (the pieces' sums added over the shard group)."""
        out = {}
        for g, t in self.flat.items():
            v = t.detach().float().abs().sum().reshape(1) if t.numel() else torch.zeros(1, device=self.device)
            if self.shard_size > 1:
                v = v.double()
                dist.all_reduce(v, group=self.group)
            out[g] = float(v.item())
        return out


class FsdpWeightGather:
    """What ``weight_sync.sync_weights`` calls for an engine store fed by a sharded trainer: one all-gather per unit
    straight into the engine's flat buffers (reference: miles/backends/fsdp_utils/update_weight_utils.py:54-294, which
    gathers ``full_tensor()`` per parameter and passes buckets to the engine)."""

    def __init__(self, src: FsdpParamStore, dst: ParamStore):
        self.src, self.dst = src, dst

    def push(self) -> int:
        return self.src.gather_into(self.dst)

    def check_status(self) -> None:
        pass
