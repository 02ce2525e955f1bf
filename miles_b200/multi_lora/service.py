"""The multi-LoRA service loop: one base model, many adapters, each with its own data, batch size, reward and lifetime.

Per iteration: snapshot of the registry -> reconcile (create tensors and prompt streams of new adapters, save and drop
retiring ones) -> for every active adapter, in slot order: activate (its merged weights become live for trainer and
engine) -> generate *its* batch from *its* prompt stream -> train -> count the step; an adapter that has reached its
``num_step`` (given, or derived from ``num_epoch`` and its dataset) is deregistered, which saves it and frees the slot.

Reference: train_multi_lora_async.py:35-101, miles/ray/multi_lora/controller.py (``mark_batch_trained``),
miles/rollout/multi_lora/{async_rollout,data_source}.py.
"""
from __future__ import annotations

import time
from typing import Optional


def train_adapter_step(loop, ctl, sources, name: str, rollout_id: int, save_interval: Optional[int] = None) -> dict:
    """One rollout + train step of adapter ``name`` on its own prompt stream and batch size. Returns the step metrics."""
    spec = ctl.registry.get(name)
    fn, args = loop.rollout_fn, loop.args
    local = getattr(fn, "args", None)
    saved = (getattr(fn, "data_source", None), getattr(local, "rollout_batch_size", None), getattr(local, "over_sampling_batch_size", None),
             loop.actor.args.global_batch_size)
    n_prompts = max(1, (spec.rollout_batch_size or args.rollout_batch_size) // max(loop.n_rep, 1))
    try:
        if hasattr(fn, "data_source"):
            fn.data_source = sources.get(name)
        if local is not None:
            local.rollout_batch_size, local.over_sampling_batch_size = n_prompts, n_prompts
        # the optimizer step of this adapter averages over this adapter's batch, whatever the service default is
        loop.actor.args.global_batch_size = n_prompts * args.n_samples_per_prompt
        ctl.activate(name)
        loop.update_weights()
        samples, _ = loop.generate(rollout_id)
        for s in samples:
            s.metadata = dict(s.metadata or {}, adapter=name)
        if args.offload_train:
            loop.actor.wake_up()
        metrics = loop.train(rollout_id, samples)
        if args.offload_train:
            loop.actor.sleep()
    finally:
        if hasattr(fn, "data_source"):
            fn.data_source = saved[0]
        if local is not None:
            local.rollout_batch_size, local.over_sampling_batch_size = saved[1], saved[2]
        loop.actor.args.global_batch_size = saved[3]
    metrics["multi_lora/samples"] = len(samples)
    if ctl.after_train(name, rollout_id, save_interval):
        ctl.registry.deregister(name)       # reached its num_step: saved and removed at the next reconciliation
        metrics["multi_lora/retired"] = 1.0
    return metrics


def run_service(loop, ctl, sources, max_rollouts: Optional[int] = None, idle_sleep: float = 1.0, can_register: bool = True,
                log=print) -> int:
    """Runs until ``max_rollouts`` adapter steps were trained (None: forever) or, when nobody can register any more,
    until no adapter is left. Returns the number of steps trained."""
    args = loop.args
    rollout_id = loop.start_rollout_id
    trained = 0
    while max_rollouts is None or trained < max_rollouts:
        active = ctl.reconcile()
        sources.reconcile([a for a in ctl.registry.snapshot()[1] if a.name in active])
        if not active:
            if not can_register:
                break  # nothing registered and nobody can register: do not spin forever
            time.sleep(idle_sleep)
            continue
        for name in active:
            m = train_adapter_step(loop, ctl, sources, name, rollout_id, getattr(args, "save_interval", None))
            if loop.ps.rank == 0:
                log(f"[multi-lora] rollout {rollout_id} adapter {name}: samples {m['multi_lora/samples']} "
                    f"loss {m.get('train/pg_loss', float('nan')):.4f} grad_norm {m.get('train/grad_norm', 0):.3f}"
                    + (" (retired)" if m.get("multi_lora/retired") else ""))
            rollout_id += 1
            trained += 1
            if max_rollouts is not None and trained >= max_rollouts:
                break
    ctl.reconcile()
    return trained
