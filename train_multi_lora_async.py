"""Multi-LoRA training service: many adapters on one base model, registered and removed while the service runs.

    python train_multi_lora_async.py --model-preset qwen3-4B --multi-lora-n-adapters 8 --multi-lora-api-port 8068 ...
    curl -X POST localhost:8068/adapters -d '{"name": "math-a", "rank": 16, "lr": 1e-4}'
    curl -X DELETE localhost:8068/adapters/math-a

``--multi-lora-adapter NAME PATH`` (repeatable) registers adapters at start-up (PATH: a PEFT directory or "none");
``--multi-lora-disable-service-mode`` runs without the HTTP API and stops when no adapter is left.

Loop (``miles_b200/multi_lora/service.py``): snapshot of the registry -> reconcile (create / retire adapter tensors and
prompt streams) -> for every active adapter: activate (merged weights become live for trainer and engine) -> generate its
batch from its own prompt stream (``prompt_data``, ``rollout_batch_size``, ``rm_type`` of the adapter's registration) ->
train -> periodic adapter save; an adapter that reaches its ``num_step`` / ``num_epoch`` is saved and removed.
Reference: train_multi_lora_async.py:35-101.
"""
from __future__ import annotations

import threading


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
    from miles_b200.multi_lora import AdapterDataSources, run_service

    sources = AdapterDataSources(args, loop.tokenizer, lambda a, tok: loop._build_data_source_for(a), registry,
                                 default_batch=args.rollout_batch_size)
    run_service(loop, ctl, sources, max_rollouts=args.num_rollout, idle_sleep=float(getattr(args, "multi_lora_idle_poll_s", 1.0) or 1.0),
                can_register=port is not None)


if __name__ == "__main__":
    main()
