"""Checkpoints of the sharded backend in the reshardable atom format of ``checkpoint/dist_ckpt.py``.

A rank's shards do not line up with parameters, let alone with atoms (a piece is ``1 / shard_size`` of a unit's flat
range). Saving therefore walks the units: each unit of the weights and of every optimizer-state part is all-gathered, and
the rank that owns the unit (``unit index mod shard size``, on the first replica) keeps host copies of its atoms; the
``torch.distributed.checkpoint`` writer then stores every rank's atoms in parallel. Loading walks the units too: every
rank reads the unit's atoms into a full-size host buffer and keeps its piece. Because the keys are the same atoms the
other trainer backend writes, either backend (under any tensor / expert / pipeline layout) loads what the other saved.

Reference: miles/backends/fsdp_utils/checkpoint.py:78-250 (``iter_%07d/{model,optimizer,lr_scheduler}`` through
``torch.distributed.checkpoint``).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

PARTS = ("m", "v", "lo", "master")


def _unit_atoms(store, u, fulls: dict, prefix: str) -> dict:
    """Atom key -> view into the full (padded) buffers of unit ``u``."""
    from ..checkpoint.dist_ckpt import param_atoms

    out = {}
    for s in u.specs:
        buf = fulls.get(s.group)
        if buf is None:
            continue
        a = s.offset - u.lo[s.group]
        t = buf[a:a + s.numel].view(s.shape)
        for key, idx in param_atoms(store, s.name):
            out[prefix + key] = t[idx] if idx else t
    return out


def state_parts(actor, with_optimizer: bool, osd: Optional[dict] = None) -> tuple:
    """``[(key prefix, {group: flat tensor laid out like the shards})]`` and the optimizer state dict they view."""
    store = actor.store
    parts = [("model.", dict(store.flat))]
    opt = getattr(actor, "opt", None)
    if with_optimizer and opt is not None and hasattr(opt, "state_dict"):
        osd = osd if osd is not None else opt.state_dict()
        for part in PARTS:
            flats = {g: st[part] for g, st in osd.items() if isinstance(st, dict) and isinstance(st.get(part), torch.Tensor)
                     and st[part].numel() == store.flat[g].numel()}
            if flats:
                parts.append((f"optim.{part}.", flats))
    return parts, osd


@torch.no_grad()
def gathered_atoms(actor, with_optimizer: bool = True) -> dict:
    """Collective. Host copies of the atoms this rank writes (weights, then optimizer state)."""
    store = actor.store
    writes = store.mesh.replicate.rank == 0
    sd = {}
    parts, _ = state_parts(actor, with_optimizer)
    for prefix, flats in parts:
        for u, fulls in store.full_units(flats):
            if writes and u.index % store.shard_size == store.shard_rank:
                for k, v in _unit_atoms(store, u, fulls, prefix).items():
                    sd[k] = v.detach().cpu().clone()
    return sd


@torch.no_grad()
def load_units(actor, directory: str, meta_keys: set, with_optimizer: bool, osd: Optional[dict]) -> bool:
    """Fill this rank's pieces of the weights (and of the optimizer state found in the checkpoint) unit by unit. Returns
    whether optimizer state was loaded (the caller then hands ``osd`` back to the optimizer)."""
    import torch.distributed.checkpoint as dcp

    store = actor.store
    parts, osd = state_parts(actor, with_optimizer, osd)
    no_dist = not (dist.is_available() and dist.is_initialized())
    S, r = store.shard_size, store.shard_rank
    loaded_optim = False
    for u in store.units:
        want, staged, fulls_by_part = {}, {}, []
        for prefix, flats in parts:
            fulls = {g: torch.zeros(u.padded[g], dtype=f.dtype) for g, f in flats.items() if u.padded[g]}
            atoms = _unit_atoms(store, u, fulls, prefix)
            missing = [k for k in atoms if k not in meta_keys]
            if missing:
                if prefix == "model.":
                    raise KeyError(f"checkpoint {directory} lacks weight atoms this model needs, e.g. {missing[:3]}")
                continue  # this part of the optimizer state was not saved (or in another form): keep what is there
            fulls_by_part.append((prefix, flats, fulls))
            for k, v in atoms.items():
                staged[k] = v
                want[k] = v if v.is_contiguous() else v.contiguous()
        if want:
            dcp.load(want, checkpoint_id=directory, no_dist=no_dist)
        for k, v in staged.items():
            if want[k].data_ptr() != v.data_ptr():
                v.copy_(want[k])  # atoms that are strided views were read into contiguous copies
        for prefix, flats, fulls in fulls_by_part:
            loaded_optim |= prefix != "model."
            for g, full in fulls.items():
                n = u.padded[g] // S
                flats[g][u.shard_off[g]:u.shard_off[g] + n].copy_(full[r * n:(r + 1) * n])
    store.invalidate()
    return loaded_optim
