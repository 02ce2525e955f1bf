"""Multi-LoRA training service: many adapters on one base model, registered and removed while the service runs.

    python train_multi_lora_async.py --model-preset qwen3-4B --multi-lora-n-adapters 8 --multi-lora-api-port 8068 ...
    curl -X POST localhost:8068/adapters -d '{"name": "math-a", "rank": 16, "lr": 1e-4}'
    curl -X DELETE localhost:8068/adapters/math-a

``--multi-lora-adapter NAME PATH`` (repeatable) registers adapters at start-up (PATH: a PEFT directory or "none");
``--multi-lora-disable-service-mode`` runs without the HTTP API and stops when no adapter is left.

Loop: snapshot of the registry -> reconcile (create / retire adapter tensors) -> for every active adapter:
activate (merged weights become live for trainer and engine) -> generate -> train -> periodic adapter save.
Reference: train_multi_lora_async.py:35-101.
"""
from __future__ import annotations

import threading
import time


def _serve(app, port: int) -> threading.Thread:
    import uvicorn

    server = uvicorn.Server(uvicorn.Config(app, host="0.0.0.0", port=port, log_level="warning"))
    t = threading.Thread(target=server.run, daemon=True)
    t.start()
    return t


def main(argv=None) -> None:
    from miles_b200.loop import RLLoop
    from miles_b200.multi_lora import AdapterRegistry, AdapterSpec, MultiLoRAController, build_control_app
    from miles_b200.utils.arguments import parse_args

    args = parse_args(argv)
    loop = RLLoop(args)
    gbs = args.global_batch_size or args.rollout_batch_size * args.n_samples_per_prompt
    registry = AdapterRegistry(max_slots=getattr(args, "multi_lora_n_adapters", 0) or 8,
                               max_adapter_batch=getattr(args, "multi_lora_max_adapter_global_batch_size", None) or 4 * gbs,
                               samples_per_prompt=args.n_samples_per_prompt)
    # an adapter's step starts once its batch is full, or after the coalesce wait on what is ready; a generate call that
    # sees no finished group at all within the empty wait fails instead of blocking the other adapters
    args.rollout_coalesce_wait_s = float(getattr(args, "multi_lora_max_coalesce_wait_s", 0.5) or 0.0)
    args.rollout_empty_wait_s = float(getattr(args, "multi_lora_max_empty_wait_s", 30.0) or 0.0)
    ctl = MultiLoRAController(loop.actor, registry, save_dir=getattr(args, "save", None))
    for name, path in getattr(args, "multi_lora_adapters", None) or []:
        registry.register(AdapterSpec(name=name, rank=getattr(args, "lora_rank", 16) or 16, alpha=getattr(args, "lora_alpha", 32) or 32,
                                      lr=args.lr, load=None if path in ("none", "") else path))
    service = getattr(args, "multi_lora_service_mode", True) is not False
    port = getattr(args, "multi_lora_api_port", None) if service else None
    if port and loop.ps.rank == 0:
        _serve(build_control_app(registry), int(port))
    rollout_id = loop.start_rollout_id
    idle_sleep = float(getattr(args, "multi_lora_idle_poll_s", 1.0) or 1.0)
    max_rollouts = args.num_rollout
    while max_rollouts is None or rollout_id < max_rollouts:
        active = ctl.reconcile()
        if not active:
            time.sleep(idle_sleep)
            if max_rollouts is not None and port is None:
                break  # nothing registered and nobody can register: do not spin forever
            continue
        for name in active:
            ctl.activate(name)
            loop.update_weights()
            samples, _ = loop.generate(rollout_id)
            for s in samples:
                s.metadata = dict(s.metadata or {}, adapter=name)
            metrics = loop.train(rollout_id, samples)
            ctl.after_train(name, rollout_id, getattr(args, "save_interval", None))
            if loop.ps.rank == 0:
                print(f"[multi-lora] rollout {rollout_id} adapter {name}: "
                      f"loss {metrics.get('train/pg_loss', float('nan')):.4f} grad_norm {metrics.get('train/grad_norm', 0):.3f}", flush=True)
            rollout_id += 1
            if max_rollouts is not None and rollout_id >= max_rollouts:
                break
    ctl.reconcile()


if __name__ == "__main__":
    main()
