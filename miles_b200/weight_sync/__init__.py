"""Trainer -> rollout-engine weight update.

Session protocol of the reference (miles/backends/megatron_utils/update_weight/mixin.py:309-389):
``pause_generation(mode) -> flush_cache (not for in_place) -> begin -> buckets -> update_weight_version ->
end -> continue_generation``.  Modes here:

* **shared**    — colocated engine running on the trainer's own ``ParamStore``: nothing is copied, the update is
  the version bump (the B200-first answer to CUDA-IPC bucket passing).
* **copy**      — engine with its own store in the same process: flat-buffer device copies; an engine that holds all
  experts next to an expert-parallel trainer receives them by all-gather (``reshard.gather_experts_into``), an engine
  next to a pipelined trainer by per-stage broadcasts (``reshard.gather_stages_into``); engines that serve MXFP8 /
  NVFP4 copies re-quantise afterwards.
* **broadcast** — engines in other processes: ``broadcast.BroadcastWeightUpdater`` (a process group that exists only
  for weight updates; buckets announced over HTTP, tensors broadcast from the trainer's source rank).
* **disk**      — ``disk_delta``: versioned XOR / overwrite deltas that engines pull.

* **push**      — an engine store that carries a ``weight_pusher``: the replica of an expert-parallel trainer is filled by
  one kernel per flat buffer that reshards, optionally quantises and stores into every GPU's replica over NVLink
  (``p2p_push.WeightPusher``, ``csrc/weight_push.cu``); the engine of a sharded (``--train-backend fsdp``) trainer by one
  all-gather per unit straight into its flat buffers (``fsdp.store.FsdpWeightGather``).
"""
from __future__ import annotations

import time
from typing import Sequence

import torch


def sync_weights(actor, engines: Sequence, mode: str | None = None) -> dict:
    args = actor.args
    t0 = time.perf_counter()
    pause_mode = getattr(args, "pause_generation_mode", "retract")
    moved = 0
    pushers = []
    for e in engines:
        e.pause_generation(pause_mode)
        if pause_mode != "in_place":
            e.flush_cache()
    t_paused = time.perf_counter()
    for e in engines:
        if e.store is actor.store:
            continue  # shared memory: nothing to move
        with torch.no_grad():
            if getattr(actor.store, "pp_size", 1) > 1 and getattr(e.store, "pp_size", 1) == 1:
                from .reshard import gather_stages_into

                moved += gather_stages_into(actor.store, e.store, actor.ps.pp)
                continue
            pusher = getattr(e.store, "weight_pusher", None)
            if pusher is not None:
                # reshard (+ quantise) + peer-memory stores + version flag in one kernel per flat buffer
                moved += pusher.push()
                pushers.append(pusher)
                continue
            for g, t in e.store.flat.items():
                src = actor.store.flat[g]
                if src.data_ptr() == t.data_ptr() and src.numel() == t.numel():
                    continue  # this group is shared
                if g == "expert" and e.store.ep_size == 1 and actor.store.ep_size > 1:
                    from .reshard import gather_experts_into

                    moved += gather_experts_into(actor.store, e.store, actor.ps.ep.group)
                    continue
                if src.numel() == t.numel():
                    t.copy_(src.to(t.dtype), non_blocking=True)
                    moved += src.numel() * src.element_size()
                else:
                    from .reshard import reshard_into

                    moved += reshard_into(actor.store, e.store, g)
    for e in engines:
        refresh = getattr(getattr(e, "model", None), "refresh_block_scaled", None)
        if refresh is not None:
            refresh()  # engines that serve MXFP8 / NVFP4 copies re-quantise from the weights that just arrived
    if actor.on_gpu:
        torch.cuda.synchronize()
    for p in pushers:
        p.check_status()  # a source that never arrived: raise rather than serve stale weights
    version = actor.store.version
    for e in engines:
        e.update_weight_version(version)
        e.continue_generation()
    t1 = time.perf_counter()
    if getattr(args, "check_weight_update_equal", False):
        check_engines_hold_trainer_weights(actor, engines)
    if getattr(args, "check_lora_weight_equal", False) and getattr(actor, "lora", None) is not None:
        for e in engines:
            actor.lora.check_merged(e.store.params)
    return {"perf/update_weights_time": t1 - t_paused, "perf/update_weights_total_time": t1 - t0,
            "perf/update_weights_bytes": moved, "weight_version": version}


def check_engines_hold_trainer_weights(actor, engines: Sequence) -> None:
    """``--check-weight-update-equal``: after an update every engine parameter of the same shape must equal the
    trainer's. ``--check-weight-update-skip-list`` (regular expressions over parameter names) leaves tensors out,
    ``--check-weight-update-selector`` picks the model (``target``/``all``: the policy; ``draft`` has nothing to check:
    no speculative draft model is served), ``--check-weight-update-allow-quant-error`` widens the tolerance to what a
    block-scaled copy of the weights may differ by."""
    import re

    args = actor.args
    if getattr(args, "check_weight_update_selector", "all") == "draft":
        return
    skip = [re.compile(p) for p in (getattr(args, "check_weight_update_skip_list", None) or [])]
    rtol = 6e-2 if getattr(args, "check_weight_update_allow_quant_error", False) else 1e-3
    for e in engines:
        if not skip:
            a, b = actor.store.checksum(), e.store.checksum()
            for g in a:
                if e.store.flat[g].numel() == actor.store.flat[g].numel():
                    assert abs(a[g] - b[g]) <= rtol * max(1.0, abs(a[g])), f"weight update mismatch in group {g}: {a[g]} vs {b[g]}"
            continue
        for name, p in actor.store.params.items():
            q = e.store.params.get(name)
            if q is None or q.shape != p.shape or any(r.search(name) for r in skip):
                continue
            sa, sb = float(p.float().abs().sum()), float(q.float().abs().sum())
            assert abs(sa - sb) <= rtol * max(1.0, abs(sa)), f"weight update mismatch in {name}: {sa} vs {sb}"
