"""Checkpoints: native sharded format, HF safetensors import / export, resume bookkeeping.

Layouts (reference: miles/backends/megatron_utils/checkpoint.py:100-198, hf_export.py:40-193,
backends/fsdp_utils/checkpoint.py:78-250):

* native : ``<dir>/iter_%07d/rank_%05d.pt`` (flat parameter buffers + optimizer state + RNG of one rank)
  and ``meta.json``; ``<dir>/latest_checkpointed_iteration.txt`` names the newest iteration — the same
  directory conventions as Megatron ``torch_dist`` so resume logic (``start_rollout_id = iteration + 1``)
  and tooling carry over.
* HF     : sharded ``model-%05d-of-%05d.safetensors`` + ``model.safetensors.index.json`` + ``config.json``
  and a ``.complete`` marker written last.
"""
from __future__ import annotations

import json
import os
import shutil
from typing import Optional

import torch
import torch.distributed as dist

from ..models.hf_mapping import from_hf, hf_names

LATEST = "latest_checkpointed_iteration.txt"


def iter_dir(base: str, iteration: int) -> str:
    return os.path.join(base, f"iter_{iteration:07d}")


def is_native_checkpoint(path: str) -> bool:
    return os.path.exists(os.path.join(path, LATEST)) or os.path.basename(os.path.normpath(path)).startswith("iter_")


def latest_iteration(base: str) -> Optional[int]:
    p = os.path.join(base, LATEST)
    if not os.path.exists(p):
        return None
    txt = open(p).read().strip()
    return int(txt) if txt.isdigit() else None


_ASYNC: dict = {"thread": None, "error": None}


def wait_for_async_save() -> None:
    """Block until a background save (``--async-save``) has finished; re-raise what it raised."""
    t = _ASYNC["thread"]
    if t is not None:
        t.join()
        _ASYNC["thread"] = None
    if _ASYNC["error"] is not None:
        err, _ASYNC["error"] = _ASYNC["error"], None
        raise RuntimeError("asynchronous checkpoint save failed") from err


def _snapshot_state(actor, iteration: int) -> dict:
    """Host copies of everything a rank saves (the device is free to move on once this returns)."""
    state = {
        "flat": {g: t.detach().cpu() for g, t in actor.store.flat.items()},
        "version": actor.store.version,
        "global_step": actor.global_step,  # optimizer steps taken (drives the LR schedule and metrics)
        "rollout_id": iteration,           # the rollout this checkpoint was written after (the directory name)
        "rng": {"cpu": torch.get_rng_state(), "cuda": torch.cuda.get_rng_state() if actor.on_gpu else None},
        "ep": (actor.store.ep_size, actor.store.ep_rank),
    }
    if actor.opt is not None and not getattr(actor.args, "no_save_optim", False):
        sd = actor.opt.state_dict()
        state["optimizer"] = {k: ({a: (b.detach().cpu() if isinstance(b, torch.Tensor) else b) for a, b in v.items()}
                                  if isinstance(v, dict) else v) for k, v in sd.items()}
    if getattr(actor, "_value_head", None) is not None:
        state["value_head"] = actor._value_head.detach().cpu()
    state["audit"] = _audit_state(actor)
    return state


def _audit_state(actor) -> dict:
    """Witness table / allocator and the event log's sequence number: a resumed run keeps counting where it stopped."""
    out = {}
    if getattr(actor, "witness", None) is not None:
        out["witness"] = actor.witness.state_dict()
    if getattr(actor, "events", None) is not None:
        out["events"] = actor.events.state_dict()
    return out


def _load_audit_state(actor, state: dict) -> None:
    if getattr(actor, "witness", None) is not None and state.get("witness") is not None:
        actor.witness.load_state_dict(state["witness"])
    if getattr(actor, "events", None) is not None and state.get("events") is not None:
        actor.events.load_state_dict(state["events"])


def _write_state(actor, base: str, d: str, iteration: int, state: dict, checksums: Optional[dict]) -> None:
    rank = actor.ps.rank
    tmp = os.path.join(d, f"rank_{rank:05d}.pt.tmp")
    torch.save(state, tmp)
    os.replace(tmp, os.path.join(d, f"rank_{rank:05d}.pt"))
    if checksums is not None:
        with open(os.path.join(d, f"weight_checksum_rank_{rank:05d}.json"), "w") as f:
            json.dump(checksums, f)


def _finish_save(actor, base: str, d: str, iteration: int) -> None:
    """After every rank has written its file: metadata, the latest pointer, retention, the post-save hook."""
    args = actor.args
    if actor.ps.rank == 0:
        meta = {}
        mp = os.path.join(d, "meta.json")
        if os.path.exists(mp):  # the reshardable format has already written its own fields
            meta = json.load(open(mp))
        meta.update({"iteration": iteration, "world_size": actor.ps.world_size, "model": actor.cfg.to_dict()})
        with open(mp, "w") as f:
            json.dump(meta, f, default=str)
        with open(os.path.join(base, LATEST), "w") as f:
            f.write(str(iteration))
        prune_checkpoints(base, iteration, getattr(args, "save_interval", None), getattr(args, "save_retain_interval", None))
    hook = getattr(args, "custom_megatron_post_save_hook_path", None)
    if hook:
        from ..utils.misc import load_function

        load_function(hook)(args, actor, iteration, d)


def prune_checkpoints(base: str, newest: int, save_interval: Optional[int], retain_interval: Optional[int]) -> list:
    """``--save-retain-interval R``: of the checkpoints older than the newest keep those whose step (rollout id + 1) is
    a multiple of R and delete the rest (reference: miles/backends/megatron_utils/checkpoint.py). Returns what was
    deleted."""
    if not retain_interval:
        return []
    gone = []
    for name in sorted(os.listdir(base)):
        if not name.startswith("iter_") or not name[5:].isdigit():
            continue
        it = int(name[5:])
        if it >= newest or (it + 1) % retain_interval == 0:
            continue
        shutil.rmtree(os.path.join(base, name), ignore_errors=True)
        gone.append(it)
    return gone


def _save_dist(actor, base: str, d: str, iteration: int) -> str:
    """``--ckpt-format torch_dist`` (default): a reshardable ``torch.distributed.checkpoint`` directory (dist_ckpt.py);
    RNG state and the value head, which are per rank, go next to it."""
    from . import dist_ckpt
    from ..utils.ci_checks import save_model_hashes

    save_model_hashes(actor.args, actor.store, actor.ps, iteration)
    side = {"rng": {"cpu": torch.get_rng_state(), "cuda": torch.cuda.get_rng_state() if actor.on_gpu else None}}
    if getattr(actor, "_value_head", None) is not None:
        side["value_head"] = actor._value_head.detach().cpu()
    side["audit"] = _audit_state(actor)
    torch.save(side, os.path.join(d, f"side_rank_{actor.ps.rank:05d}.pt"))
    fut = dist_ckpt.save(actor, d, iteration, async_save=bool(getattr(actor.args, "async_save", False)))
    if fut is not None:
        import threading

        def work():
            try:
                fut.result()
                _finish_save(actor, base, d, iteration)
            except BaseException as e:  # noqa: BLE001 - surfaced by wait_for_async_save
                _ASYNC["error"] = e

        t = threading.Thread(target=work, name="miles-b200-async-save", daemon=False)
        _ASYNC["thread"] = t
        t.start()
        return d
    if dist.is_initialized():
        dist.barrier()
    _finish_save(actor, base, d, iteration)
    return d


def save_checkpoint(actor, base: str, iteration: int) -> str:
    """One file per rank under ``<base>/iter_%07d``. With ``--async-save`` the device-to-host snapshot happens here and
    the file write, metadata, retention and hooks run in a background thread (the next save, or the end of the run,
    waits for it); ranks then synchronise through the files themselves instead of a barrier."""
    wait_for_async_save()
    d = iter_dir(base, iteration)
    os.makedirs(d, exist_ok=True)
    if getattr(actor.args, "ckpt_format", "torch_dist") == "torch_dist":
        return _save_dist(actor, base, d, iteration)
    state = _snapshot_state(actor, iteration)
    checksums = None
    if getattr(actor.args, "save_local_weight_checksum", False):
        checksums = {g: float(t.double().abs().sum()) for g, t in state["flat"].items()}
    from ..utils.ci_checks import save_model_hashes

    save_model_hashes(actor.args, actor.store, actor.ps, iteration)
    if getattr(actor.args, "async_save", False):
        import threading
        import time

        def work():
            try:
                _write_state(actor, base, d, iteration, state, checksums)
                if actor.ps.rank == 0:  # every rank's file must exist before the checkpoint is announced
                    deadline = time.time() + 600
                    want = [os.path.join(d, f"rank_{r:05d}.pt") for r in range(actor.ps.world_size)]
                    while not all(os.path.exists(w) for w in want):
                        if time.time() > deadline:
                            raise TimeoutError(f"rank files missing under {d}")
                        time.sleep(0.05)
                _finish_save(actor, base, d, iteration)
            except BaseException as e:  # noqa: BLE001 - surfaced by wait_for_async_save
                _ASYNC["error"] = e

        t = threading.Thread(target=work, name="miles-b200-async-save", daemon=False)
        _ASYNC["thread"] = t
        t.start()
        return d
    _write_state(actor, base, d, iteration, state, checksums)
    if dist.is_initialized():
        dist.barrier()
    _finish_save(actor, base, d, iteration)
    return d


def load_checkpoint(actor, path: str, step: Optional[int] = None) -> Optional[int]:
    """Load a native checkpoint or an HF directory. A native checkpoint returns the rollout id it was written
    after (the ``iter_`` number; training resumes at the next one) and restores ``actor.global_step``, the count of
    optimizer steps, which differs from the rollout id whenever a rollout takes several optimizer steps. An HF
    directory, or ``--finetune``, returns None (start from rollout 0)."""
    if is_native_checkpoint(path):
        it = step if step is not None else latest_iteration(path)
        d = iter_dir(path, it) if it is not None else path
        from . import dist_ckpt

        if dist_ckpt.is_dist_checkpoint(d):
            return _load_dist(actor, d, it)
        f = os.path.join(d, f"rank_{actor.ps.rank:05d}.pt")
        state = torch.load(f, map_location="cpu", weights_only=False)
        with torch.no_grad():
            for g, t in actor.store.flat.items():
                t.copy_(state["flat"][g].to(t.dtype))
        actor.store.version = state.get("version", 0)
        if actor.opt is not None and "optimizer" in state and not getattr(actor.args, "no_load_optim", False):
            actor.opt.load_state_dict(state["optimizer"])
        elif actor.opt is not None:
            actor.opt.sync_master_from_params()
        if not getattr(actor.args, "no_load_rng", False) and "rng" in state:
            torch.set_rng_state(state["rng"]["cpu"])
        if getattr(actor, "_value_head", None) is not None and "value_head" in state:
            actor._value_head.data.copy_(state["value_head"])
        _load_audit_state(actor, state.get("audit") or {})
        from ..utils.ci_checks import check_model_hashes

        if it is not None:
            check_model_hashes(actor.args, actor.store, actor.ps, it)
        if getattr(actor.args, "finetune", False):
            return None
        actor.global_step = int(state.get("global_step", 0) or 0)
        rid = state.get("rollout_id", it)
        return int(rid) if rid is not None else None
    if os.path.isdir(path):
        import contextlib

        # a sharded store keeps what is written into its per-unit views only inside writing()
        with (actor.store.writing(gather=False) if getattr(actor.store, "is_fsdp", False) else contextlib.nullcontext()):
            load_hf(actor.cfg, actor.store, path)
        if actor.opt is not None:
            actor.opt.sync_master_from_params()
        return None
    raise FileNotFoundError(f"checkpoint {path} not found")


def _load_dist(actor, d: str, it: Optional[int]) -> Optional[int]:
    from . import dist_ckpt
    from ..utils.ci_checks import check_model_hashes

    with_opt = actor.opt is not None and not getattr(actor.args, "no_load_optim", False)
    meta = dist_ckpt.load(actor, d, with_optimizer=with_opt)
    actor.store.version = int(meta.get("version", 0) or 0)
    if actor.opt is not None and not with_opt:
        actor.opt.sync_master_from_params()
    side_p = os.path.join(d, f"side_rank_{actor.ps.rank:05d}.pt")
    if os.path.exists(side_p):  # same layout as the run that saved: per-rank extras apply
        side = torch.load(side_p, map_location="cpu", weights_only=False)
        if not getattr(actor.args, "no_load_rng", False) and side.get("rng"):
            torch.set_rng_state(side["rng"]["cpu"])
        if getattr(actor, "_value_head", None) is not None and "value_head" in side:
            actor._value_head.data.copy_(side["value_head"])
        _load_audit_state(actor, side.get("audit") or {})
    if it is not None:
        check_model_hashes(actor.args, actor.store, actor.ps, it)
    if getattr(actor.args, "finetune", False):
        return None
    actor.global_step = int(meta.get("global_step", 0) or 0)
    rid = meta.get("rollout_id", it)
    return int(rid) if rid is not None else None


def load_weights_into_backup(actor, tag: str, path: str, step: Optional[int] = None) -> None:
    """Load a checkpoint into the pinned host copy ``tag`` without disturbing the live weights."""
    actor.backup_weights("_tmp_live")
    load_checkpoint(actor, path, step)
    actor.backup_weights(tag)
    actor.restore_weights("_tmp_live")
    del actor.weights_backup["_tmp_live"]


# ------------------------------------------------------------------ HuggingFace safetensors
def load_hf(cfg, store, path: str, strict: bool = True) -> int:
    from safetensors import safe_open

    idx = os.path.join(path, "model.safetensors.index.json")
    if os.path.exists(idx):
        wm = json.load(open(idx))["weight_map"]
        files = sorted(set(wm.values()))
    else:
        files = sorted(f for f in os.listdir(path) if f.endswith(".safetensors"))
        wm = None
    handles = {f: safe_open(os.path.join(path, f), framework="pt", device="cpu") for f in files}
    where = dict(wm) if wm else {k: f for f, h in handles.items() for k in h.keys()}

    def get(name):
        f = where.get(name)
        return handles[f].get_tensor(name) if f is not None else None

    return from_hf(cfg, store, get, strict)


def export_hf(actor, out_dir: str, max_shard_bytes: int = 5 << 30, tokenizer_dir: Optional[str] = None) -> str:
    """Collective export of the live weights in HF layout; each rank writes its own shards."""
    from safetensors.torch import save_file

    cfg, store, ps = actor.cfg, actor.store, actor.ps
    os.makedirs(out_dir, exist_ok=True)
    marker = os.path.join(out_dir, ".complete")
    if ps.rank == 0 and os.path.exists(marker):
        os.remove(marker)
    shards, cur, size = [], {}, 0
    for hf_name, t in hf_names(cfg, store, tp_group=ps.tp.group if ps.tp.size > 1 else None):
        is_expert = ".experts." in hf_name
        if getattr(store, "is_fsdp", False) and ps.rank != 0:
            continue  # every rank of a sharded trainer sees the same gathered tensors: the first one writes them
        if ps.tp.size > 1 and ps.tp.rank != 0:
            continue  # the gathered tensors are identical on every tensor-parallel rank
        if not is_expert and ps.dp_cp.rank != 0:
            continue  # replicated tensors are written once
        if hf_name == "model.embed_tokens.weight" and ps.pp.size > 1 and ps.pp.rank != 0:
            continue  # a tied embedding also lives on the last pipeline stage (as its LM head)
        nb = t.numel() * t.element_size()
        if cur and size + nb > max_shard_bytes:
            shards.append(cur)
            cur, size = {}, 0
        cur[hf_name] = t.detach().contiguous().cpu()
        if getattr(store, "is_fsdp", False) and cur[hf_name].device == t.device:
            cur[hf_name] = cur[hf_name].clone()  # the unit buffers are reused: keep a copy, not a view
        size += nb
    if cur:
        shards.append(cur)
    counts = [len(shards)]
    if dist.is_initialized() and ps.world_size > 1:
        gathered = [None] * ps.world_size
        dist.all_gather_object(gathered, len(shards))
        counts = gathered
    total = sum(counts)
    first = sum(counts[:ps.rank])
    weight_map = {}
    for j, sh in enumerate(shards):
        fname = f"model-{first + j + 1:05d}-of-{total:05d}.safetensors"
        save_file(sh, os.path.join(out_dir, fname), metadata={"format": "pt"})
        for k in sh:
            weight_map[k] = fname
    maps = [weight_map]
    if dist.is_initialized() and ps.world_size > 1:
        maps = [None] * ps.world_size
        dist.all_gather_object(maps, weight_map)
    if ps.rank == 0:
        merged = {}
        for m in maps:
            merged.update(m)
        nbytes = sum(p.numel() * p.element_size() for p in store.flat.values())
        with open(os.path.join(out_dir, "model.safetensors.index.json"), "w") as f:
            json.dump({"metadata": {"total_size": nbytes}, "weight_map": merged}, f, indent=1)
        with open(os.path.join(out_dir, "config.json"), "w") as f:
            json.dump(cfg.to_hf_config(), f, indent=1)
        src = tokenizer_dir or getattr(actor.args, "hf_checkpoint", None)
        if src and os.path.isdir(src):
            for fn in os.listdir(src):
                if fn.startswith("tokenizer") or fn in ("vocab.json", "merges.txt", "special_tokens_map.json", "generation_config.json"):
                    shutil.copy(os.path.join(src, fn), os.path.join(out_dir, fn))
    if dist.is_initialized():
        dist.barrier()
    if ps.rank == 0:
        open(marker, "w").write("ok")
    return out_dir


def is_complete_hf_dir(path: str) -> bool:
    return os.path.exists(os.path.join(path, ".complete"))
