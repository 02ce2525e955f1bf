"""Weight update by peer-memory push: reshard + (optionally) quantise + store into the engines' buffers in one kernel.

``--update-weight-transfer-mode p2p`` of the reference moves trainer shards to the engines with RDMA writes planned
once per (source shard, target engine) pair (miles/backends/megatron_utils/update_weight/update_weight_from_distributed/
p2p.py, broadcast.py:201-291, with the MXFP8 / NVFP4 post-processing of processors/quantizer_mxfp8.py:6-116 and
quantizer_nvfp4.py:36-203). On one NVSwitch node the same job is a kernel: every GPU maps the engines' weight
buffers (CUDA IPC, ``parallel/symm.py``) and ``csrc/weight_push.cu`` reads the local shard once and stores it, already
in the engine's layout and number format, into every engine GPU that needs it, then raises a version flag there.

Planning uses the checkpoint *atoms* (``checkpoint/dist_ckpt.py``): the pieces of a parameter that no supported layout
splits (one expert, one KV-head group of the fused QKV, one column group of the output projection, one slab of the
FFN width). An atom held by a trainer shard and needed by an engine shard is one 2-D slab of the kernel's table, so
every (tensor-, expert-parallel) trainer layout maps onto every engine layout with the same code. When several
trainer ranks hold an atom (replicated parameters, data-parallel replicas) the engine's own GPU sends it if it can
(a local copy), else the lowest rank that holds it.

Buffers that receive pushes live in one ``SymmetricRegion`` per GPU (``PushTarget``): the engine's bf16 parameter
store (``flat_override`` of ``ParamStore``), and / or block-scaled copies (values + scale-factor atoms of
``ops/mx_gemm.MxOperand``) that the push quantises into directly.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Sequence

import torch
import torch.distributed as dist

from ..checkpoint.dist_ckpt import param_atoms
from ..models import ParamStore
from ..ops import _ext

MODES = {"bf16": 0, "mxfp8": 1, "nvfp4": 2}
MX_SUFFIXES = ("attn.qkv.weight", "attn.o.weight", "mlp.gate_up.weight", "mlp.down.weight", "moe.w1", "moe.w2")


def _slab(shape: Sequence[int], idx: tuple) -> tuple:
    """(row0, col0, rows, cols, ld) of ``tensor[idx]`` in the 2-D view ``[prod(shape[:-1]), shape[-1]]``."""
    shape = list(shape) if len(shape) > 1 else [1, int(shape[0])]
    K = int(shape[-1])
    R = 1
    for d in shape[:-1]:
        R *= int(d)
    if idx == ():
        return 0, 0, R, K, K
    first = idx[0]
    if isinstance(first, int):              # one expert of [E, rows, K]
        per = R // int(shape[0])
        return first * per, 0, per, K, K
    if first == slice(None):                # a column range
        c = idx[1]
        return 0, int(c.start), R, int(c.stop - c.start), K
    if len(shape) == 2 and shape[0] == 1 and len(idx) == 1:  # a range of a vector (bias)
        return 0, int(first.start), 1, int(first.stop - first.start), K
    return int(first.start), 0, int(first.stop - first.start), K, K


def _join_adjacent(rows: list) -> list:
    """Join slabs that continue one another in source and destination (same tensor, same destinations): column-wise
    neighbours of equal height first (the slabs of one FFN width, the head groups of the output projection), then
    row-wise neighbours of equal width (head groups of the fused QKV, consecutive experts). Fewer, larger slabs; and
    a joined slab satisfies the block alignment of the quantised formats where a single atom may not."""
    # row = [src_off, rows, cols, src_ld, tensor, dst_row0, dst_col0, mask]
    rows = sorted(rows, key=lambda r: (r[4], r[7], r[5], r[6]))
    out = []
    for r in rows:
        p = out[-1] if out else None
        if (p is not None and p[4] == r[4] and p[7] == r[7] and p[5] == r[5] and p[1] == r[1] and p[3] == r[3]
                and p[6] + p[2] == r[6] and p[0] + p[2] == r[0]):
            p[2] += r[2]
        else:
            out.append(list(r))
    out.sort(key=lambda r: (r[4], r[7], r[6], r[5]))
    res = []
    for r in out:
        p = res[-1] if res else None
        if (p is not None and p[4] == r[4] and p[7] == r[7] and p[6] == r[6] and p[2] == r[2] and p[3] == r[3]
                and p[5] + p[1] == r[5] and p[0] + p[1] * p[3] == r[0]):
            p[1] += r[1]
        else:
            res.append(list(r))
    return res


@dataclass
class PushTarget:
    """The receiving side on one GPU: a symmetric region that holds the engine store's flat buffers (``groups``) and /
    or block-scaled copies of the matrices named by ``quant`` (``"mxfp8"`` / ``"nvfp4"``)."""
    region: object
    store: Optional[ParamStore]
    flat_off: dict = field(default_factory=dict)          # group -> byte offset of the flat buffer inside the region
    mx: dict = field(default_factory=dict)                # parameter name -> MxOperand (values / atoms inside the region)
    mx_off: dict = field(default_factory=dict)            # parameter name -> (values offset, atoms offset)
    quant: str = "none"
    flag_off: int = 0
    flags_addr: int = 0
    amax: Optional[torch.Tensor] = None                   # nvfp4: one slot per quantised tensor
    amax_slot: dict = field(default_factory=dict)

    @staticmethod
    def region_bytes(cfg, dtype, groups: Sequence[str], quant: str, tp_size: int = 1, ep_size: int = 1) -> int:
        meta = ParamStore(cfg, "cpu", dtype, ep_size=ep_size, tp_size=tp_size, meta=True, init=False)
        n = 4096
        for g in groups:
            n += meta.sizes[g] * 2 + 512
        if quant != "none":
            for s in meta.specs:
                if s.name.endswith(MX_SUFFIXES):
                    rows, K = s.numel // s.shape[-1], s.shape[-1]
                    per = 32 if quant == "mxfp8" else 16
                    n += (rows * K if quant == "mxfp8" else rows * K // 2) + ((rows + 127) // 128) * ((K // per + 3) // 4) * 512 + 1024
        return n

    @classmethod
    def create(cls, cfg, ps_group, rank: int, world: int, device, dtype=torch.bfloat16, groups: Sequence[str] = ("expert",),
               quant: str = "none", tp_size: int = 1, tp_rank: int = 0, ep_size: int = 1, ep_rank: int = 0,
               share_dense: Optional[ParamStore] = None, build_store: bool = True) -> "PushTarget":
        """Collective over ``ps_group``: allocates and exchanges the region, carves the buffers at identical offsets on
        every rank. ``groups``: the flat buffers of the engine store that live in the region (pushed as bf16)."""
        from ..ops.mx_gemm import MxOperand
        from ..parallel.symm import SymmetricRegion

        assert dtype == torch.bfloat16, "the push kernel reads and writes bf16 weights"
        nbytes = cls.region_bytes(cfg, dtype, groups if build_store else (), quant, tp_size, ep_size)
        region = SymmetricRegion(nbytes, ps_group, rank, world, device)
        flags, _ = region.carve((8,), torch.int64)
        flags.zero_()
        t = cls(region=region, store=None, quant=quant)
        t.flag_off = flags.data_ptr() - region.base
        t.flags_addr = flags.data_ptr()
        meta = ParamStore(cfg, "cpu", dtype, ep_size=ep_size, ep_rank=ep_rank, tp_size=tp_size, tp_rank=tp_rank, meta=True, init=False)
        override = {}
        if build_store:
            for g in groups:
                buf, _ = region.carve((meta.sizes[g],), dtype)
                buf.zero_()
                override[g] = buf
                t.flat_off[g] = buf.data_ptr() - region.base
            t.store = ParamStore(cfg, device, dtype, ep_size=ep_size, ep_rank=ep_rank, tp_size=tp_size, tp_rank=tp_rank, init=False,
                                 share_dense=share_dense if "dense" not in groups else None, flat_override=override)
        if quant != "none":
            per = 32 if quant == "mxfp8" else 16
            names = [s for s in meta.specs if s.name.endswith(MX_SUFFIXES)]
            t.amax = torch.zeros(max(len(names), 1), dtype=torch.float32, device=device)
            for i, s in enumerate(names):
                rows, K = s.numel // s.shape[-1], s.shape[-1]
                step = 128 if quant == "mxfp8" else 256
                if K % step or rows % 128:
                    continue
                q, _ = region.carve((rows, K if quant == "mxfp8" else K // 2), torch.uint8)
                atoms, _ = region.carve(((rows + 127) // 128, (K // per + 3) // 4, 512), torch.uint8)
                atoms.zero_()
                t.amax_slot[s.name] = i
                dec = 1.0
                op = MxOperand(quant, q, torch.empty(0, dtype=torch.uint8, device=device), atoms, dec, t.amax[i:i + 1] if quant == "nvfp4" else None)
                t.mx[s.name] = op
                t.mx_off[s.name] = (q.data_ptr() - region.base, atoms.data_ptr() - region.base)
        torch.cuda.synchronize(device)
        dist.barrier(group=ps_group)
        return t

    def finish_nvfp4(self) -> None:
        """After a push: per-tensor decode scales of the NVFP4 copies from the amax the push used."""
        if self.quant != "nvfp4":
            return
        for name, op in self.mx.items():
            a = self.amax[self.amax_slot[name]:self.amax_slot[name] + 1]
            op.decode_scale = torch.where(a > 0, a / (448.0 * 6.0), torch.ones_like(a))


@dataclass
class Layout:
    """How one rank shards the model (what ``ParamStore`` needs to know)."""
    tp_size: int = 1
    tp_rank: int = 0
    ep_size: int = 1
    ep_rank: int = 0

    def meta_store(self, cfg) -> ParamStore:
        return ParamStore(cfg, "cpu", torch.bfloat16, ep_size=self.ep_size, ep_rank=self.ep_rank, tp_size=self.tp_size,
                          tp_rank=self.tp_rank, meta=True, init=False)


class WeightPusher:
    """One rank's sender (and receiver bookkeeping) of the peer-memory weight update.

    ``src_store``: this rank's trainer shard. ``trainer_layouts[r]`` / ``engine_layouts[r]``: the layout of rank ``r``'s
    trainer shard and of the engine shard hosted on rank ``r``'s GPU (``None``: no engine there). ``target``: this
    rank's ``PushTarget`` (every rank's region has the same carving). ``skip_groups``: flat groups the engine shares
    with the trainer by address (nothing to move)."""

    def __init__(self, cfg, src_store: ParamStore, target: PushTarget, rank: int, trainer_layouts: Sequence[Layout],
                 engine_layouts: Sequence[Optional[Layout]], skip_groups: Sequence[str] = (), amax_group=None, wait_ms: float = 2000.0,
                 barrier_first: bool = True):
        self.C = _ext.load(required=True)
        self.cfg, self.src, self.target, self.rank = cfg, src_store, target, rank
        self.world = len(trainer_layouts)
        self.amax_group = amax_group
        self.wait_ms = wait_ms
        self.barrier_first = barrier_first
        dev = src_store.device
        self.counter = torch.zeros(1, dtype=torch.int32, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self.version = 0
        # who holds which atom, and where
        t_meta = [l.meta_store(cfg) for l in trainer_layouts]
        e_meta = [l.meta_store(cfg) if l is not None else None for l in engine_layouts]
        holders: dict[str, list] = {}
        for r, st in enumerate(t_meta):
            for s in st.specs:
                for key, _ in param_atoms(st, s.name):
                    holders.setdefault(key, []).append(r)
        my = t_meta[rank]
        tensors, t_index = [], {}
        segs = {g: [] for g in ("dense", "expert")}
        self.sources_of = [set() for _ in range(self.world)]   # destination rank -> source ranks
        e_ref = next(m for m in e_meta if m is not None)
        for r, em in enumerate(e_meta):
            if em is None:
                continue
            for s in em.specs:
                if s.group in skip_groups:
                    continue
                for key, didx in param_atoms(em, s.name):
                    hs = holders.get(key)
                    assert hs, f"no trainer rank holds {key}"
                    srcr = r if r in hs else hs[0]
                    self.sources_of[r].add(srcr)
                    if srcr != rank:
                        continue
                    sidx = dict(param_atoms(my, s.name))[key]
                    ms = my.by_name[s.name]
                    sr0, sc0, rows, cols, sld = _slab(ms.shape, sidx)
                    dr0, dc0, drows, dcols, dld = _slab(s.shape, didx)
                    assert (rows, cols) == (drows, dcols), (key, rows, cols, drows, dcols)
                    src_off = ms.offset + sr0 * sld + sc0
                    for mode in self._modes_for(s, target):
                        tk = (s.name, mode)
                        if tk not in t_index:
                            t_index[tk] = len(tensors)
                            tensors.append(self._tensor_row(e_ref.by_name[s.name], mode, dld))
                        segs[ms.group].append([src_off, rows, cols, sld, t_index[tk], dr0, dc0, 1 << r])
        # slabs that differ only in the destination rank become one slab with a wider mask (the shard is read once)
        self.tables = {}
        for g, rows_ in segs.items():
            merged: dict[tuple, int] = {}
            for sg in rows_:
                k = tuple(sg[:7])
                merged[k] = merged.get(k, 0) | sg[7]
            if not merged:
                continue
            tab = torch.tensor(_join_adjacent([list(k) + [m] for k, m in merged.items()]), dtype=torch.int64)
            for row in tab.tolist():
                mode = tensors[row[4]][3]
                need = {0: 8, 1: 128, 2: 64}[mode]
                assert row[0] % 8 == 0 and row[3] % 8 == 0 and row[2] % need == 0 and row[6] % need == 0, \
                    f"slab {row} is not aligned for mode {mode}"
            self.tables[g] = (tab.to(dev), int((tab[:, 1] * tab[:, 2] // 8).sum()))
        self.tensors = torch.tensor(tensors if tensors else [[0] * 8], dtype=torch.int64, device=dev)
        self.flag_mask = 0
        for r in range(self.world):
            if rank in self.sources_of[r]:
                self.flag_mask |= 1 << r
        self.src_mask = 0
        for s_ in self.sources_of[rank]:
            self.src_mask |= 1 << s_
        # bf16 bytes read from the shard times the number of destinations (what crosses NVLink or is copied locally)
        self.bytes_pushed = 0
        for tab, _ in self.tables.values():
            for row in tab.tolist():
                self.bytes_pushed += row[1] * row[2] * 2 * bin(row[7]).count("1")

    # ------------------------------------------------------------------ tables
    @staticmethod
    def _modes_for(spec, target: PushTarget) -> list:
        modes = []
        if target.store is not None and spec.group in target.flat_off:
            modes.append(0)
        if target.quant != "none" and spec.name in target.mx:
            modes.append(MODES[target.quant])
        return modes

    def _tensor_row(self, espec, mode: int, dld: int) -> list:
        t = self.target
        if mode == 0:
            return [t.flat_off[espec.group] + espec.offset * 2, 0, dld, 0, 0, 0, 0, 0]
        q_off, a_off = t.mx_off[espec.name]
        return [q_off, a_off, espec.shape[-1], mode, t.amax_slot[espec.name], 0, 0, 0]

    # ------------------------------------------------------------------ the update
    @torch.no_grad()
    def push(self, version: Optional[int] = None) -> int:
        """Send this rank's share of the update and wait (bounded, on the device) for the shares of the others.
        Every rank calls it once per update. Returns the bytes this rank stored (all destinations)."""
        self.version = int(version) if version is not None else self.version + 1
        t = self.target
        if self.barrier_first and dist.is_initialized():
            # nobody stores into an engine that may still be reading its weights: every rank has paused its engine
            # (the caller does that before calling) once all ranks are here
            dist.barrier(group=self.amax_group)
        amax = None
        if t.quant == "nvfp4":
            # one scale per destination tensor: max |w| over every trainer shard of it
            t.amax.zero_()
            for name, slot in t.amax_slot.items():
                if name in self.src.params:
                    t.amax[slot] = self.src.params[name].abs().max().float()
            dist.all_reduce(t.amax, op=dist.ReduceOp.MAX, group=self.amax_group)
            amax = t.amax
        bases = [int(b) for b in t.region.peer_base]
        for g, (tab, nvec) in self.tables.items():
            self.C.weight_push(self.src.flat[g], tab, self.tensors, amax, bases, t.flag_off, self.rank, 0, self.version, self.counter, nvec)
        # the flags go up after the last table: an empty table that only raises the flags
        self.C.weight_push(self.src.flat["dense"], self._flag_only_table(), self.tensors, amax, bases, t.flag_off, self.rank,
                           self.flag_mask, self.version, self.counter, 1)
        if self.src_mask:
            self.C.weight_push_wait(t.flags_addr, self.src_mask, self.version, self.wait_ms, self.status)
        t.finish_nvfp4()
        return self.bytes_pushed

    def _flag_only_table(self) -> torch.Tensor:
        if not hasattr(self, "_flag_tab"):
            self._flag_tab = torch.zeros(1, 8, dtype=torch.int64, device=self.src.device)  # zero rows: nothing is copied
        return self._flag_tab

    def check_status(self) -> None:
        code = int(self.status.item())
        if code:
            self.status.zero_()
            raise RuntimeError(f"weight push: a source rank's update never arrived (status {code}); the engine weights are stale")
