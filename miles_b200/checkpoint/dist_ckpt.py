"""Reshardable checkpoints in the ``torch.distributed.checkpoint`` format (``--ckpt-format torch_dist``).

A checkpoint written under one parallel layout must load under another (the reference gets this from Megatron's
``torch_dist`` format, miles/backends/megatron_utils/checkpoint.py:100-176). Here every parameter is cut into *atoms*,
the largest pieces that no supported layout ever splits, and each atom is one entry of a DCP state dict under a key
that names it globally:

* an expert tensor ``layers.i.moe.w1`` [E_local, 2I, H]  ->  one atom per global expert, ``...moe.w1.e17``;
* the fused ``attn.qkv.weight`` / ``bias``               ->  per global KV head ``h``: its query-head rows ``.q{h}``,
                                                            key rows ``.k{h}``, value rows ``.v{h}``;
* ``attn.o.weight``                                      ->  the input columns of KV head group ``h``: ``.c{h}``;
* ``mlp.gate_up.weight`` / ``mlp.down.weight``           ->  eight slabs of the FFN width: ``.g{c}`` / ``.u{c}`` / ``.c{c}``;
* everything else (norms, router, embeddings)            ->  one atom, the parameter's own name.

A rank saves the atoms it holds; atoms that several ranks hold (replicated parameters) are written once (DCP removes
duplicate keys while planning). A rank loads the atoms its layout needs, whichever rank wrote them, so tensor-, expert-
and pipeline-parallel sizes may all differ between save and load. Optimizer state uses the same atoms under the
prefixes ``optim.m.``, ``optim.v.`` and ``optim.lo.`` / ``optim.master.`` (the fp32 master as 16-bit remainder or as
fp32). ``save`` can run in the background (``--async-save``, ``torch.distributed.checkpoint.async_save``).
"""
from __future__ import annotations

import json
import os
from typing import Iterator, Optional

import torch
import torch.distributed as dist

FFN_SLABS = 8


def param_atoms(store, name: str) -> Iterator[tuple]:
    """Yield ``(atom_key, index)`` for the local tensor of ``name``: ``local[index]`` is the atom (a view)."""
    cfg, g = store.cfg, store.global_cfg
    tp, tr = store.tp_size, store.tp_rank
    spec = store.by_name[name]
    D = g.head_dim
    if spec.group == "expert":
        el = cfg.num_experts // store.ep_size
        for le in range(el):
            yield f"{name}.e{store.ep_rank * el + le}", (le,)
        return
    if name.endswith(("attn.qkv.weight", "attn.qkv.bias")):
        G = g.num_q_heads // g.num_kv_heads
        hk_local = g.num_kv_heads // tp
        ql, kl = hk_local * G * D, hk_local * D
        for j in range(hk_local):
            h = tr * hk_local + j
            yield f"{name}.q{h}", (slice(j * G * D, (j + 1) * G * D),)
            yield f"{name}.k{h}", (slice(ql + j * D, ql + (j + 1) * D),)
            yield f"{name}.v{h}", (slice(ql + kl + j * D, ql + kl + (j + 1) * D),)
        return
    if name.endswith("attn.o.weight"):
        G = g.num_q_heads // g.num_kv_heads
        hk_local = g.num_kv_heads // tp
        for j in range(hk_local):
            yield f"{name}.c{tr * hk_local + j}", (slice(None), slice(j * G * D, (j + 1) * G * D))
        return
    if name.endswith(("mlp.gate_up.weight", "mlp.down.weight")) and g.ffn_hidden_size % FFN_SLABS == 0 and FFN_SLABS % tp == 0:
        I_loc = g.ffn_hidden_size // tp
        w = g.ffn_hidden_size // FFN_SLABS
        per = FFN_SLABS // tp
        for j in range(per):
            c = tr * per + j
            if name.endswith("gate_up.weight"):
                yield f"{name}.g{c}", (slice(j * w, (j + 1) * w),)
                yield f"{name}.u{c}", (slice(I_loc + j * w, I_loc + (j + 1) * w),)
            else:
                yield f"{name}.c{c}", (slice(None), slice(j * w, (j + 1) * w))
        return
    assert tp == 1 or not name.endswith(("mlp.gate_up.weight", "mlp.down.weight")), \
        f"{name}: the FFN width must divide into {FFN_SLABS} slabs for a tensor-parallel checkpoint"
    yield name, ()


def _views(store, flat_by_group: dict, prefix: str) -> dict:
    """Atoms of per-parameter views into flat buffers laid out like the parameters (weights or optimizer state)."""
    out = {}
    for s in store.specs:
        flat = flat_by_group.get(s.group)
        if flat is None:
            continue
        t = flat[s.offset:s.offset + s.numel].view(s.shape)
        for key, idx in param_atoms(store, s.name):
            out[prefix + key] = t[idx] if idx else t
    return out


def state_atoms(actor, with_optimizer: bool = True, osd: Optional[dict] = None) -> dict:
    """The DCP state dict of this rank: atom key -> tensor view (weights, then optimizer state). ``osd``: an optimizer
    state dict to take the views from (default: a fresh ``opt.state_dict()``)."""
    store = actor.store
    sd = _views(store, store.flat, "model.")
    opt = getattr(actor, "opt", None)
    if with_optimizer and opt is not None and hasattr(opt, "state_dict"):
        osd = osd if osd is not None else opt.state_dict()
        for part in ("m", "v", "lo", "master"):
            flats = {g: st[part] for g, st in osd.items() if isinstance(st, dict) and st.get(part) is not None
                     and isinstance(st[part], torch.Tensor) and st[part].numel() == store.flat[g].numel()}
            sd.update(_views(store, flats, f"optim.{part}."))
    return sd


def save(actor, directory: str, iteration: int, async_save: bool = False):
    """Write ``directory`` (one ``iter_`` folder). Returns the future of an asynchronous save, else None."""
    import torch.distributed.checkpoint as dcp

    os.makedirs(directory, exist_ok=True)
    with_opt = not getattr(actor.args, "no_save_optim", False)
    if getattr(actor.store, "is_fsdp", False):
        from ..fsdp.checkpoint import gathered_atoms

        # a sharded store: units are gathered and every rank keeps host copies of the atoms of the units it owns
        sd = gathered_atoms(actor, with_opt)
    else:
        sd = {k: v.detach() for k, v in state_atoms(actor, with_opt).items()}
        if async_save:
            sd = {k: v.cpu().clone() for k, v in sd.items()}  # the device may move on: the writer thread owns host copies
    opt = getattr(actor, "opt", None)
    extra = {"iteration": iteration, "global_step": actor.global_step, "rollout_id": iteration, "version": actor.store.version,
             "optimizer_step": getattr(opt, "step_count", 0) if opt is not None else 0, "model": actor.cfg.to_dict(),
             "saved_layout": {"tp": actor.store.tp_size, "ep": actor.store.ep_size, "pp": actor.store.pp_size,
                              "world": actor.ps.world_size, "fsdp_shards": getattr(actor.store, "shard_size", 0)}}
    if actor.ps.rank == 0:
        with open(os.path.join(directory, "meta.json"), "w") as f:
            json.dump(extra, f, default=str)
    no_dist = not (dist.is_available() and dist.is_initialized())
    if async_save and not no_dist:
        return dcp.async_save(sd, checkpoint_id=directory)
    dcp.save(sd, checkpoint_id=directory, no_dist=no_dist)
    return None


def load(actor, directory: str, with_optimizer: bool = True) -> dict:
    """Fill this rank's weights (and optimizer state, where the checkpoint has it) from ``directory``, whatever layout
    wrote it. Returns the checkpoint's ``meta.json``."""
    import torch.distributed.checkpoint as dcp
    from torch.distributed.checkpoint import FileSystemReader

    meta_keys = set(FileSystemReader(directory).read_metadata().state_dict_metadata.keys())
    opt = getattr(actor, "opt", None)
    # resident optimizer state is handed out as the live tensors; state kept in pinned host chunks as concatenated host
    # copies, which are loaded here and written back through load_state_dict below
    osd = opt.state_dict() if (with_optimizer and opt is not None and hasattr(opt, "state_dict")) else {}
    if getattr(actor.store, "is_fsdp", False):
        from ..fsdp.checkpoint import load_units

        if load_units(actor, directory, meta_keys, with_optimizer, osd or None):
            opt.load_state_dict(osd)
        else:
            osd = {}
        return _finish_load(actor, directory, bool(osd))
    want = state_atoms(actor, with_optimizer, osd or None)
    sd = {}
    for k, v in want.items():
        if k not in meta_keys:
            continue
        sd[k] = v if v.is_contiguous() else v.contiguous()
    missing = [k for k in want if k.startswith("model.") and k not in meta_keys]
    if missing:
        raise KeyError(f"checkpoint {directory} lacks {len(missing)} weight atoms this layout needs, e.g. {missing[:3]}")
    no_dist = not (dist.is_available() and dist.is_initialized())
    dcp.load(sd, checkpoint_id=directory, no_dist=no_dist)
    with torch.no_grad():
        for k, v in want.items():  # non-contiguous views were loaded into contiguous copies
            if k in sd and sd[k].data_ptr() != v.data_ptr():
                v.copy_(sd[k])
    got_optim = bool(osd) and any(k.startswith("optim.") for k in sd)
    if got_optim:
        # state_dict() hands out the live tensors for resident state; offloaded chunks were concatenated into copies
        opt.load_state_dict(osd)
    return _finish_load(actor, directory, got_optim)


def _finish_load(actor, directory: str, got_optim: bool) -> dict:
    opt = getattr(actor, "opt", None)
    meta = {}
    p = os.path.join(directory, "meta.json")
    if os.path.exists(p):
        meta = json.load(open(p))
    if got_optim and hasattr(opt, "step_count"):
        opt.step_count = int(meta.get("optimizer_step", opt.step_count))
    return meta


def is_dist_checkpoint(directory: str) -> bool:
    return os.path.exists(os.path.join(directory, ".metadata"))
