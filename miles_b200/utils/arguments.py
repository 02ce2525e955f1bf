"""Command-line surface of ``train.py`` / ``train_async.py`` / ``train_multi_lora_async.py``.

The parser is assembled from three sources so that launch scripts written for the reference keep
working:

1. ``flag_table.FLAG_GROUPS`` — the framework's own flag groups (cluster, train, rollout, data, eval,
   algo, lora, debug, ...), names and defaults as in miles/utils/arguments.py:106-2589;
2. ``TRAINER_FLAGS`` — the subset of Megatron-LM model/optimizer/parallelism flags that the reference's
   launchers actually pass (shape flags, ``--tensor-model-parallel-size``, ``--lr-decay-style`` ...); the
   trainer here consumes them directly instead of forwarding to Megatron;
3. engine passthrough — every ``--sglang-<name>`` / ``--eval-sglang-<name>`` option is accepted and
   collected into ``args.sglang_*`` (mirrors miles/backends/sglang_utils/arguments.py:110-207); the
   in-process engine reads the ones it implements (mem fraction, max running requests, cuda-graph
   batch sizes, page size, chunked prefill size ...).

``validate_args`` performs the cross-flag checks and derivations of ``miles_validate_args``
(miles/utils/arguments.py:2848-3523) that apply to this backend and rejects features that are not
built rather than ignoring them silently.
"""
from __future__ import annotations

import argparse
import json
import os
import re
from typing import Any, Optional, Sequence

from .flag_table import FLAG_GROUPS

_KIND = {"i": int, "f": float, "s": str, "j": json.loads}

# (flag, kind, default, extra) — Megatron-LM flags consumed natively by this trainer
TRAINER_FLAGS = [
    # parallelism
    ("--tensor-model-parallel-size", "i", 1, {}), ("--pipeline-model-parallel-size", "i", 1, {}),
    ("--context-parallel-size", "i", 1, {}), ("--expert-model-parallel-size", "i", 1, {}),
    ("--expert-tensor-parallel-size", "i", None, {}), ("--sequence-parallel", "b", False, {}),
    ("--virtual-pipeline-model-parallel-size", "i", None, {}), ("--cp-comm-type", "s", "p2p", {"choices": ["p2p", "a2a", "allgather"]}),
    ("--decoder-first-pipeline-num-layers", "i", None, {}), ("--decoder-last-pipeline-num-layers", "i", None, {}),
    ("--use-distributed-optimizer", "B", True, {}), ("--overlap-grad-reduce", "B", True, {}),
    ("--overlap-param-gather", "B", True, {}), ("--accumulate-allreduce-grads-in-fp32", "b", False, {}),
    # model shape
    ("--num-layers", "i", None, {}), ("--hidden-size", "i", None, {}), ("--ffn-hidden-size", "i", None, {}),
    ("--num-attention-heads", "i", None, {}), ("--group-query-attention", "b", False, {}),
    ("--num-query-groups", "i", None, {}), ("--kv-channels", "i", None, {}), ("--vocab-size", "i", None, {}),
    ("--make-vocab-size-divisible-by", "i", 128, {}), ("--normalization", "s", "RMSNorm", {}),
    ("--norm-epsilon", "f", 1e-6, {}), ("--swiglu", "b", False, {}), ("--disable-bias-linear", "b", False, {}),
    ("--add-qkv-bias", "b", False, {}), ("--qk-layernorm", "b", False, {}),
    ("--untie-embeddings-and-output-weights", "b", False, {}), ("--position-embedding-type", "s", "rope", {}),
    ("--use-rotary-position-embeddings", "b", False, {}), ("--rotary-base", "f", 1e6, {}),
    ("--rotary-percent", "f", 1.0, {}), ("--max-position-embeddings", "i", 40960, {}), ("--seq-length", "i", 4096, {}),
    ("--attention-softmax-in-fp32", "b", False, {}), ("--attention-backend", "s", "flash", {}),
    ("--attention-dropout", "f", 0.0, {}), ("--hidden-dropout", "f", 0.0, {}), ("--transformer-impl", "s", "native", {}),
    ("--spec", "s", None, {"nargs": "+"}), ("--no-rope-fusion", "b", False, {}), ("--no-masked-softmax-fusion", "b", False, {}),
    ("--no-gradient-accumulation-fusion", "b", False, {}), ("--attention-output-gate", "b", False, {}),
    ("--apply-layernorm-1p", "b", False, {}),
    # GLM-4 dense: sandwich norms and checkpoints with interleaved rotary rows
    ("--post-self-attn-layernorm", "b", False, {}), ("--post-mlp-layernorm", "b", False, {}), ("--rotary-interleaved", "b", False, {}),
    # MoE
    ("--num-experts", "i", None, {}), ("--moe-router-topk", "i", 2, {}), ("--moe-ffn-hidden-size", "i", None, {}),
    ("--moe-layer-freq", "s", "1", {}), ("--moe-router-score-function", "s", "softmax", {}),
    ("--moe-router-pre-softmax", "b", False, {}), ("--moe-router-dtype", "s", "fp32", {}),
    ("--moe-router-load-balancing-type", "s", "none", {}), ("--moe-aux-loss-coeff", "f", 0.0, {}),
    ("--moe-grouped-gemm", "b", False, {}), ("--moe-token-dispatcher-type", "s", "alltoall", {}),
    ("--moe-permute-fusion", "b", False, {}), ("--moe-router-enable-expert-bias", "b", False, {}),
    ("--moe-router-bias-update-rate", "f", 0.0, {}), ("--moe-router-topk-scaling-factor", "f", None, {}),
    ("--moe-shared-expert-intermediate-size", "i", None, {}), ("--moe-shared-expert-gate", "b", False, {}),
    ("--moe-enable-deepep", "b", False, {}), ("--moe-token-drop-policy", "s", "probs", {}),
    ("--moe-router-num-groups", "i", None, {}), ("--moe-router-group-topk", "i", None, {}),
    ("--moe-router-padding-for-quantization", "b", False, {}), ("--moe-latent-size", "i", None, {}),
    # MLA (accepted for shape files; rejected by the validator until the model family is built)
    ("--multi-latent-attention", "b", False, {}), ("--q-lora-rank", "i", None, {}), ("--kv-lora-rank", "i", None, {}),
    ("--qk-head-dim", "i", None, {}), ("--v-head-dim", "i", None, {}), ("--qk-pos-emb-head-dim", "i", None, {}),
    ("--rotary-scaling-factor", "f", None, {}), ("--use-rope-scaling", "b", False, {}), ("--mscale", "f", None, {}),
    ("--mscale-all-dim", "f", None, {}), ("--original-max-position-embeddings", "i", None, {}),
    ("--beta-fast", "f", None, {}), ("--beta-slow", "f", None, {}), ("--no-position-embedding", "b", False, {}),
    # optimizer / schedule
    ("--rollout-quantization", "s", "none", {"choices": ["none", "mxfp8", "nvfp4"]}),
    ("--rollout-engine-urls", "s", None, {}), ("--rollout-prefill-urls", "s", None, {}), ("--launch-rollout-fleet", "b", False, {}), ("--rollout-router-url", "s", None, {}), ("--sglang-config", "s", None, {}), ("--rollout-fleet-device", "s", None, {}),
    ("--rollout-fleet-base-port", "i", 30000, {}),
    ("--custom-agent-function-path", "s", None, {}), ("--tito-family", "s", None, {"choices": ["chatml", "qwen3", "llama3", "generic"]}),
    ("--muon-momentum", "f", 0.95, {}), ("--muon-num-ns-steps", "i", 5, {}), ("--muon-extra-scale-factor", "f", 1.0, {}),
    ("--muon-scale-mode", "s", "spectral", {"choices": ["spectral", "unit_rms_norm"]}),
    ("--muon-no-nesterov", "b", False, {}), ("--muon-no-split-qkv", "b", False, {}),
    ("--optimizer", "s", "adam", {"choices": ["adam", "sgd", "muon"]}), ("--lr", "f", 1e-6, {}), ("--min-lr", "f", 0.0, {}),
    ("--lr-decay-style", "s", "constant", {"choices": ["constant", "linear", "cosine", "WSD"]}),
    ("--lr-warmup-iters", "i", 0, {}), ("--lr-decay-iters", "i", None, {}), ("--lr-wsd-decay-iters", "i", None, {}),
    ("--lr-warmup-fraction", "f", None, {}), ("--weight-decay", "f", 0.1, {}), ("--adam-beta1", "f", 0.9, {}),
    ("--adam-beta2", "f", 0.98, {}), ("--adam-eps", "f", 1e-8, {}), ("--clip-grad", "f", 1.0, {}),
    ("--use-precision-aware-optimizer", "b", False, {}), ("--optimizer-cpu-offload", "b", False, {}),
    ("--overlap-cpu-optimizer-d2h-h2d", "b", False, {}), ("--exp-avg-dtype", "s", "fp32", {"choices": ["fp32", "bf16", "fp16", "fp8"]}),
    ("--exp-avg-sq-dtype", "s", "fp32", {"choices": ["fp32", "bf16", "fp16", "fp8"]}),
    ("--main-params-dtype", "s", "fp32", {"choices": ["fp32", "bf16"]}), ("--offload-optimizer-states", "b", False, {}),
    # precision
    ("--bf16", "b", True, {}), ("--fp16", "b", False, {}), ("--fp8-format", "s", None, {}), ("--fp8-recipe", "s", None, {}),
    ("--fp8-param-gather", "b", False, {}), ("--fp4-format", "s", None, {}), ("--te-precision-config-file", "s", None, {}),
    ("--num-layers-at-start-in-bf16", "i", 0, {}), ("--num-layers-at-end-in-bf16", "i", 0, {}),
    ("--reuse-grad-buf-for-mxfp8-param-ag", "b", False, {}),
    # memory / recompute
    ("--recompute-granularity", "s", "full", {"choices": ["full", "selective", "none"]}),
    ("--recompute-method", "s", "uniform", {}), ("--recompute-num-layers", "i", 1, {}),
    # checkpoint / misc
    ("--ckpt-format", "s", "torch_dist", {"choices": ["torch_dist", "torch"]}),
    ("--load", "s", None, {}), ("--save", "s", None, {}), ("--save-interval", "i", None, {}), ("--ckpt-step", "i", None, {}),
    ("--save-retain-interval", "i", None, {}), ("--async-save", "b", False, {}), ("--no-save-optim", "b", False, {}),
    ("--no-load-optim", "b", False, {}), ("--no-load-rng", "b", False, {}), ("--finetune", "b", False, {}),
    ("--seed", "i", 1234, {}), ("--global-batch-size", "i", None, {}), ("--micro-batch-size", "i", 1, {}),
    ("--calculate-per-token-loss", "b", False, {}), ("--distributed-backend", "s", "nccl", {}),
    ("--distributed-timeout-minutes", "i", 10, {}), ("--eval-interval", "i", None, {}), ("--low-memory-resume", "b", False, {}),
    ("--mtp-num-layers", "i", None, {}), ("--mtp-loss-scaling-factor", "f", 0.2, {}), ("--custom-config-path", "s", None, {}),
    ("--padded-vocab-size", "i", None, {}), ("--wandb-project", "s", None, {}), ("--deterministic-mode", "b", False, {}),
    ("--no-check-for-nan-in-loss-and-grad", "b", False, {}), ("--log-interval", "i", 1, {}),
    ("--tokenizer-type", "s", "HuggingFaceTokenizer", {}), ("--tokenizer-model", "s", None, {}),
    # sharded data-parallel backend (--train-backend fsdp); names of the reference's fsdp_utils/arguments.py:10-66
    ("--dp-replicate-size", "i", 1, {}), ("--fsdp-cpu-offload", "b", False, {}), ("--keep-fp32-master", "B", True, {}),
    ("--gradient-checkpointing", "b", False, {}), ("--fsdp-state-dict-cpu-offload", "B", True, {}),
    ("--config", "s", None, {}), ("--fsdp-num-unit-buffers", "i", 2, {}),
    # destroy the trainer's NCCL sub-groups while the colocated engine generates, rebuild them before training
    ("--reload-process-groups", "b", False, {}),
    # run dashboard (names of the reference's miles/dashboard/args.py); telemetry is collected whenever --dump-details is set
    ("--use-miles-dashboard", "b", False, {}), ("--dashboard-flush-interval", "f", 5.0, {}),
    ("--dashboard-gpu-sample-interval", "f", 1.0, {}), ("--dashboard-sglang-scrape-interval", "f", 2.0, {}),
    ("--dashboard-sglang-scrape-mode", "s", "auto", {"choices": ["auto", "router", "direct"]}),
    ("--dashboard-sglang-metrics", "s", None, {}), ("--dashboard-forward-prometheus", "b", False, {}),
    # host-memory samples with phase marks, written as CSV by the first rank (tools/host_memory_profiler.py)
    ("--profile-host-memory", "s", None, {}), ("--profile-host-memory-interval", "f", 0.5, {}),
    # native extensions of this framework
    ("--model-preset", "s", None, {}), ("--model-backend", "s", "auto", {"choices": ["auto", "b200", "torch"]}),
    ("--init-std", "f", 0.02, {}), ("--engine-page-size", "i", 64, {}), ("--engine-max-prefill-tokens", "i", 16384, {}),
    ("--fused-comm", "B", True, {}), ("--weight-sync-quant", "s", "none", {"choices": ["none", "mxfp8", "nvfp4", "fp8_block"]}),
    # rollout on a full replica of the experts (all-gathered at every weight update) instead of an expert-parallel engine
    ("--rollout-replicate-experts", "B", None, {}), ("--share-kv-grad-memory", "B", True, {}),
]

_UNBUILT = {
    "multi_latent_attention": "multi-latent attention models (DeepSeek / Kimi / GLM-5 families)",
}


def _add(group, flag: str, kind: str, default: Any, extra: dict) -> None:
    names = [flag] + list(extra.get("aliases", []))
    kw: dict = {}
    if "dest" in extra:
        kw["dest"] = extra["dest"]
    if kind == "b":
        group.add_argument(*names, action="store_true", default=bool(default) if default is not None else False, **kw)
    elif kind == "nb":
        group.add_argument(*names, action="store_false", default=True if default is None else default, **kw)
    elif kind == "B":
        group.add_argument(*names, action=argparse.BooleanOptionalAction, default=default, **kw)
    elif kind == "a":
        group.add_argument(*names, action="append", type=_KIND.get(extra.get("type", "s"), str), default=default, **kw)
    else:
        if "choices" in extra:
            kw["choices"] = extra["choices"]
        if "nargs" in extra:
            kw["nargs"] = extra["nargs"]
            if extra["nargs"] == "?":
                kw["const"] = extra.get("const", True)  # the bare flag switches the feature on
        group.add_argument(*names, type=_KIND[kind], default=default, **kw)


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser("miles_b200", allow_abbrev=False, conflict_handler="resolve")
    seen: set = set()
    for gname, flags in FLAG_GROUPS.items():
        g = p.add_argument_group(gname)
        for flag, kind, default, extra in flags:
            if flag in seen:
                continue
            seen.add(flag)
            _add(g, flag, kind, default, extra)
    g = p.add_argument_group("trainer")
    for flag, kind, default, extra in TRAINER_FLAGS:
        if flag in seen:
            continue
        seen.add(flag)
        _add(g, flag, kind, default, extra)
    return p


_ENGINE_RE = re.compile(r"^--(eval-)?sglang-([a-z0-9-]+)$")


def _parse_engine_passthrough(rest: Sequence[str], ns: argparse.Namespace) -> list:
    """Collect ``--sglang-x [v ...]`` / ``--eval-sglang-x`` into namespace attributes; return leftovers."""
    left, i = [], 0
    while i < len(rest):
        tok = rest[i]
        key, _, inline = tok.partition("=")
        m = _ENGINE_RE.match(key)
        if not m:
            left.append(tok)
            i += 1
            continue
        name = ("eval_" if m.group(1) else "") + "sglang_" + m.group(2).replace("-", "_")
        vals = [inline] if inline else []
        i += 1
        while not inline and i < len(rest) and not rest[i].startswith("--"):
            vals.append(rest[i])
            i += 1
        if not vals:
            v: Any = True
        else:
            conv = []
            for s in vals:
                try:
                    conv.append(json.loads(s))
                except Exception:
                    conv.append(s)
            v = conv[0] if len(conv) == 1 else conv
        setattr(ns, name, v)
    return left


def parse_args(argv: Optional[Sequence[str]] = None, validate: bool = True, add_custom_arguments=None) -> argparse.Namespace:
    parser = build_parser()
    if add_custom_arguments is not None:
        add_custom_arguments(parser)
    ns, rest = parser.parse_known_args(argv)
    left = _parse_engine_passthrough(rest, ns)
    if left:
        # user rollout / generate functions may declare extra flags through ``fn.add_arguments``
        extra_parser = argparse.ArgumentParser(add_help=False, allow_abbrev=False)
        used = _load_user_arguments(ns, extra_parser)
        if used:
            ns2, left = extra_parser.parse_known_args(left)
            for k, v in vars(ns2).items():
                setattr(ns, k, v)
        if left:
            parser.error(f"unrecognized arguments: {' '.join(left)}")
    if validate:
        validate_args(ns)
    return ns


def _load_user_arguments(ns, parser) -> bool:
    from .misc import load_function

    used = False
    for attr in ("rollout_function_path", "custom_generate_function_path", "custom_rm_path", "data_source_path"):
        path = getattr(ns, attr, None)
        if not path:
            continue
        try:
            fn = load_function(path)
        except Exception:
            continue
        adder = getattr(fn, "add_arguments", None)
        if adder is not None:
            adder(parser)
            used = True
    return used


def _default(ns, name: str, value: Any) -> None:
    if getattr(ns, name, None) is None:
        setattr(ns, name, value)


_DEFAULTS: dict = {}


def parser_defaults() -> dict:
    """dest -> default of every flag of the parser (cached)."""
    if not _DEFAULTS:
        _DEFAULTS.update({a.dest: a.default for a in build_parser()._actions})
    return _DEFAULTS


def validate_args(args: argparse.Namespace) -> argparse.Namespace:
    for attr, what in _UNBUILT.items():
        if getattr(args, attr, False):
            raise NotImplementedError(f"--{attr.replace('_', '-')}: {what} is not built in this framework yet")
    from . import flag_policy

    # flags of features that are not built raise; flags of components that do not exist here warn once
    flag_policy.apply(args, parser_defaults())
    if getattr(args, "custom_config_path", None):
        import yaml

        with open(args.custom_config_path) as f:
            for k, v in (yaml.safe_load(f) or {}).items():
                setattr(args, k, v)
    if getattr(args, "config", None):
        # the sharded backend's YAML file: keys are flag names with underscores; unknown keys are an error, not a no-op
        # (reference: fsdp_utils/arguments.py:100-123)
        import yaml

        with open(args.config) as f:
            data = yaml.safe_load(f) or {}
        unknown = sorted(k for k in data if not hasattr(args, k))
        if unknown:
            raise ValueError(f"unknown key(s) in the YAML config {args.config}: {', '.join(unknown)}")
        for k, v in data.items():
            setattr(args, k, v)
    if getattr(args, "train_backend", "megatron") == "fsdp":
        for flag in ("tensor_model_parallel_size", "pipeline_model_parallel_size", "expert_model_parallel_size"):
            if int(getattr(args, flag, 1) or 1) != 1:
                raise ValueError(f"--train-backend fsdp is data parallel only: --{flag.replace('_', '-')} must be 1")
        for flag, what in (("lora_rank", "LoRA"), ("use_fault_tolerance", "independent data-parallel cells"),
                           ("stream_optimizer_state_to_disk", "optimizer state on disk")):
            if getattr(args, flag, None):
                raise NotImplementedError(f"--train-backend fsdp with {what} (--{flag.replace('_', '-')}) is not built")
        if getattr(args, "update_weight_transfer_mode", "broadcast") == "disk-delta":
            raise NotImplementedError("--train-backend fsdp updates engines by all-gather, not through disk deltas")
        if int(getattr(args, "dp_replicate_size", 1) or 1) < 1:
            raise ValueError("--dp-replicate-size must be at least 1")
    elif int(getattr(args, "dp_replicate_size", 1) or 1) != 1 or getattr(args, "fsdp_cpu_offload", False):
        raise ValueError("--dp-replicate-size / --fsdp-cpu-offload belong to --train-backend fsdp")
    # ---- algorithm
    assert not (args.kl_coef != 0 and args.kl_loss_coef != 0), "only one of --kl-coef and --kl-loss-coef can be set"
    if args.advantage_estimator in ("reinforce_plus_plus", "reinforce_plus_plus_baseline"):
        assert args.normalize_advantages, f"{args.advantage_estimator} requires --normalize-advantages"
    if args.use_rollout_logprobs:
        assert not args.use_tis, "--use-rollout-logprobs and --use-tis are mutually exclusive"
    if args.get_mismatch_metrics:
        assert args.custom_tis_function_path is not None, "--get-mismatch-metrics needs --custom-tis-function-path"
    _default(args, "eps_clip_high", args.eps_clip)
    _default(args, "eval_reward_key", getattr(args, "reward_key", None))
    if args.use_rollout_routing_replay:
        args.use_routing_replay = True
    if getattr(args, "use_rollout_indexer_replay", False):
        args.use_indexer_replay = True
    args.use_critic = args.advantage_estimator == "ppo"
    if args.use_critic:
        assert args.kl_coef == 0, "shared actor/critic PPO does not support reward-level KL; use --use-kl-loss"
    _default(args, "critic_load", args.load)
    _default(args, "critic_lr", args.lr)
    if getattr(args, "critic_save", None) is None and args.save is not None:
        args.critic_save = args.save.rstrip("/") + "_critic"
    if (args.kl_coef != 0 or args.use_kl_loss) and args.ref_load is not None and not os.path.exists(args.ref_load):
        raise FileNotFoundError(f"ref_load {args.ref_load} does not exist")
    if args.use_opd:
        if args.opd_type is None:
            raise ValueError("--opd-type must be given with --use-opd")
        if args.opd_type == "megatron" and args.opd_teacher_load is None:
            raise ValueError("--opd-teacher-load is required with --opd-type megatron")
        if args.opd_type == "sglang":
            # teacher servers score the samples during the rollout (rollout/on_policy_distillation.py)
            from ..rollout.on_policy_distillation import parse_teacher_urls

            if args.opd_teacher_load is not None:
                raise ValueError("--opd-teacher-load belongs to --opd-type megatron; with sglang the teacher is a server")
            if not parse_teacher_urls(getattr(args, "opd_teacher_urls", None)) and not getattr(args, "rm_url", None):
                raise ValueError("--opd-type sglang needs --opd-teacher-urls NAME=URL ... or --rm-url")
            if int(getattr(args, "opd_log_prob_top_k", 0) or 0) > 0 and getattr(args, "opd_top_k_strategy", "only-student") != "only-teacher":
                raise NotImplementedError("--opd-log-prob-top-k is built for --opd-top-k-strategy only-teacher (the teacher's top-k "
                                          "per position); strategies that need the student's top-k are not")
        elif int(getattr(args, "opd_log_prob_top_k", 0) or 0) > 0 or getattr(args, "opd_teacher_urls", None):
            raise ValueError("--opd-log-prob-top-k / --opd-teacher-urls need --opd-type sglang")
    elif getattr(args, "opd_teacher_urls", None):
        raise ValueError("--opd-teacher-urls is set but --use-opd is not")
    # ---- batching
    if args.use_dynamic_batch_size:
        assert args.max_tokens_per_gpu is not None, "--use-dynamic-batch-size needs --max-tokens-per-gpu"
        _default(args, "log_probs_max_tokens_per_gpu", args.max_tokens_per_gpu)
    if args.num_steps_per_rollout is not None:
        gbs = args.rollout_batch_size * args.n_samples_per_prompt // args.num_steps_per_rollout
        if args.global_batch_size is not None:
            assert args.global_batch_size == gbs, (
                f"global_batch_size {args.global_batch_size} != rollout_batch_size*n_samples_per_prompt//num_steps_per_rollout = {gbs}")
        args.global_batch_size = gbs
    elif args.global_batch_size is None and args.rollout_batch_size is not None:
        args.global_batch_size = args.rollout_batch_size * args.n_samples_per_prompt
    if args.n_samples_per_prompt == 1:
        args.grpo_std_normalization = False
    _default(args, "over_sampling_batch_size", args.rollout_batch_size)
    assert args.over_sampling_batch_size >= args.rollout_batch_size, "--over-sampling-batch-size must be >= --rollout-batch-size"
    if args.num_epoch is None:
        assert args.num_rollout is not None, "set --num-rollout or --num-epoch"
    if args.rollout_max_context_len is not None:
        _default(args, "rollout_max_prompt_len", args.rollout_max_context_len - 1)
        assert args.rollout_max_prompt_len <= args.rollout_max_context_len - 1
    _default(args, "eval_max_context_len", args.rollout_max_context_len)
    # ---- placement / offload
    if getattr(args, "offload", False):
        args.offload_train = True
        args.offload_rollout = True
    world = args.actor_num_nodes * args.actor_num_gpus_per_node
    if args.colocate:
        _default(args, "offload_train", True)
        _default(args, "offload_rollout", True)
        args.rollout_num_gpus = world
    _default(args, "offload_train", False)
    _default(args, "offload_rollout", False)
    _default(args, "rollout_num_gpus", world)
    assert not (args.debug_rollout_only and args.debug_train_only), "--debug-rollout-only and --debug-train-only are exclusive"
    if args.load_debug_rollout_data is not None:
        args.debug_train_only = True
    if args.dump_details is not None:
        args.save_debug_rollout_data = f"{args.dump_details}/rollout_data/{{rollout_id}}.pt"
        args.save_debug_train_data = f"{args.dump_details}/train_data/{{rollout_id}}_{{rank}}.pt"
    if args.ci_test and not args.debug_rollout_only and not args.debug_train_only and not args.ci_disable_weight_update_checker:
        args.check_weight_update_equal = True
    if getattr(args, "rollout_external", False):
        # engines somebody else started (--rollout-external --rollout-external-engine-addrs host:port ...): the same
        # path as --rollout-engine-urls
        addrs = getattr(args, "rollout_external_engine_addrs", None) or []
        assert addrs, "--rollout-external needs --rollout-external-engine-addrs host:port ..."
        assert not getattr(args, "sglang_config", None) and not getattr(args, "launch_rollout_fleet", False), \
            "--rollout-external engines are not launched by the job: drop --sglang-config / --launch-rollout-fleet"
        args.rollout_engine_urls = ",".join(a if a.startswith("http") else "http://" + a for a in addrs)
        args.colocate = False
    elif getattr(args, "rollout_external_engine_addrs", None):
        raise ValueError("--rollout-external-engine-addrs is set but --rollout-external is not")
    if args.update_weight_transfer_mode in ("p2p", "disk-delta"):
        assert not args.colocate, f"--update-weight-transfer-mode {args.update_weight_transfer_mode} is not compatible with --colocate"
    if args.update_weight_transfer_mode == "disk-delta":
        assert args.update_weight_disk_dir, "disk-delta needs --update-weight-disk-dir"
    if args.save_interval is not None:
        assert args.save is not None, "--save is required with --save-interval"
    if args.lora_rank > 0:
        assert args.target_modules is not None, "--target-modules is required when LoRA is enabled"
        tm = args.target_modules
        if tm == "all-linear":
            mods = ["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"]
        else:
            mods = [m.strip() for m in tm.split(",")] if isinstance(tm, str) else list(tm)
        if args.exclude_modules:
            ex = {m.strip() for m in args.exclude_modules.split(",")}
            mods = [m for m in mods if m not in ex]
        args.target_modules = mods
    # ---- parallel layout of this trainer: DP x TP x EP on one box (PP/CP sizes are validated by the topology)
    tp, pp, cp = args.tensor_model_parallel_size, args.pipeline_model_parallel_size, args.context_parallel_size
    assert world % (tp * pp * cp) == 0, f"world size {world} is not divisible by tp*pp*cp = {tp * pp * cp}"
    args.world_size = world
    args.data_parallel_size = world // (tp * pp * cp)
    if args.sequence_parallel and tp == 1:
        args.sequence_parallel = False
    # ---- engine knobs derived from the passthrough
    _default(args, "sglang_mem_fraction_static", 0.7 if args.colocate else 0.85)
    _default(args, "sglang_max_running_requests", None)
    _default(args, "sglang_server_concurrency", 512)
    if getattr(args, "model_preset", None) or (getattr(args, "hf_checkpoint", None)
                                               and os.path.exists(os.path.join(args.hf_checkpoint, "config.json"))):
        model_config_from_args(args)  # fails now, not after the cluster is up, when the flags and the model disagree
    return args


def hf_validate_args(args, hf_config: dict) -> None:
    """When both an HF checkpoint and explicit shape flags are given they must describe the same model: compares
    every shape flag that was set against ``config.json`` and reports all mismatches at once
    (reference: miles/utils/arguments.py:3656-3707)."""
    cfg = dict(hf_config.get("text_config", hf_config))  # multimodal configs nest the language model
    rope = cfg.get("rope_parameters")
    if isinstance(rope, dict) and "rope_theta" not in cfg:
        theta = rope.get("rope_theta") or next((v["rope_theta"] for v in rope.values() if isinstance(v, dict) and "rope_theta" in v), None)
        if theta is not None:
            cfg["rope_theta"] = theta
    same = lambda a, b: a == b
    close = lambda a, b: abs(float(a) - float(b)) <= 1e-12 + 1e-6 * abs(float(b))
    table = [("hidden_size", "hidden_size", same), ("num_attention_heads", "num_attention_heads", same),
             ("num_key_value_heads", "num_query_groups", same), ("num_hidden_layers", "num_layers", same),
             ("intermediate_size", "ffn_hidden_size", same), ("moe_intermediate_size", "moe_ffn_hidden_size", same),
             ("num_experts", "num_experts", same), ("num_experts_per_tok", "moe_router_topk", same),
             ("tie_word_embeddings", "untie_embeddings_and_output_weights", lambda h, a: bool(h) != bool(a)),
             ("rms_norm_eps", "norm_epsilon", close), ("rope_theta", "rotary_base", close), ("head_dim", "kv_channels", same)]
    errors = []
    for hf_key, flag, ok in table:
        have = getattr(args, flag, None)
        if hf_key not in cfg or have is None:
            continue
        if flag == "untie_embeddings_and_output_weights" and not getattr(args, "num_layers", None):
            continue  # a store_true flag is only meaningful when the shape was given by flags at all
        if not ok(cfg[hf_key], have):
            errors.append(f"{hf_key}={cfg[hf_key]!r} in the checkpoint config but --{flag.replace('_', '-')} is {have!r}")
    if errors:
        raise AssertionError("model shape flags contradict the HF checkpoint: " + "; ".join(errors))


def _sandwich_norms(args) -> bool:
    a, b = bool(getattr(args, "post_self_attn_layernorm", False)), bool(getattr(args, "post_mlp_layernorm", False))
    if a != b:
        raise NotImplementedError("--post-self-attn-layernorm and --post-mlp-layernorm come together (GLM-4 sandwich norms)")
    if a and getattr(args, "num_experts", None):
        raise NotImplementedError("sandwich norms are built for dense MLP layers")
    return a


def _first_dense_layers(freq, num_layers: int) -> int:
    """Megatron's ``--moe-layer-freq`` as a pattern (``"[0]*1+[1]*45"`` or a list): how many leading layers are dense."""
    if isinstance(freq, str) and "[" in freq:
        pattern = eval(freq, {"__builtins__": {}})  # noqa: S307 - an arithmetic list expression from the launch script
    elif isinstance(freq, (list, tuple)):
        pattern = list(freq)
    else:
        return 0
    n = 0
    for v in pattern[:num_layers]:
        if v:
            break
        n += 1
    assert all(pattern[n:num_layers]), "--moe-layer-freq: dense layers are supported at the start of the stack only"
    return n


def _check_architecture_flags(args, cfg):
    """The model comes from a preset or a checkpoint: architecture flags that were given and say something else would
    otherwise be dropped without a word (and the job would train another model than the command line describes)."""
    moe = cfg.is_moe
    given = [("moe_router_score_function", cfg.router_score if moe else "softmax", "softmax"),
             ("moe_router_enable_expert_bias", bool(cfg.router_bias), False),
             ("moe_shared_expert_intermediate_size", cfg.shared_expert_ffn or None, None),
             ("moe_shared_expert_gate", bool(cfg.shared_expert_gate), False),
             ("moe_router_topk_scaling_factor", cfg.routed_scaling_factor if cfg.routed_scaling_factor != 1.0 else None, None),
             ("moe_router_num_groups", cfg.n_group if cfg.n_group != 1 else None, None),
             ("moe_router_group_topk", cfg.topk_group if cfg.n_group != 1 else None, None),
             ("rotary_percent", (cfg.rotary_dim or cfg.head_dim) / cfg.head_dim, 1.0),
             ("use_rope_scaling", bool(cfg.rope_scaling), False),
             ("post_self_attn_layernorm", bool(cfg.post_norms), False), ("post_mlp_layernorm", bool(cfg.post_norms), False),
             ("rotary_interleaved", bool(cfg.rope_interleaved), False)]
    bad = []
    for flag, have, default in given:
        v = getattr(args, flag, default)
        if v in (None, default) or v == have:
            continue
        if isinstance(v, float) and have is not None and abs(float(v) - float(have)) < 1e-9:
            continue
        bad.append(f"--{flag.replace('_', '-')} {v!r} (the model has {have!r})")
    if bad:
        raise NotImplementedError(f"model {cfg.name!r} does not match the architecture flags: " + "; ".join(bad) +
                                  ". The flags describe a model only together with the --num-layers / --hidden-size / ... shape flags")
    return cfg


def model_config_from_args(args):
    """Build a ``ModelConfig`` from a preset, an HF checkpoint dir, or Megatron-style shape flags."""
    from ..models.config import ModelConfig, get_config

    if getattr(args, "model_preset", None):
        return _check_architecture_flags(args, get_config(args.model_preset))
    if getattr(args, "hf_checkpoint", None) and os.path.exists(os.path.join(args.hf_checkpoint, "config.json")):
        import json

        with open(os.path.join(args.hf_checkpoint, "config.json")) as f:
            hf_validate_args(args, json.load(f))
        return _check_architecture_flags(args, ModelConfig.from_hf_config(args.hf_checkpoint))
    assert args.num_layers and args.hidden_size and args.num_attention_heads, \
        "model shape needs --model-preset, --hf-checkpoint or the --num-layers/--hidden-size/... flags"
    heads = args.num_attention_heads
    moe = bool(args.num_experts)
    return ModelConfig(
        name=getattr(args, "model_name", None) or "custom",
        num_layers=args.num_layers, hidden_size=args.hidden_size, num_q_heads=heads,
        num_kv_heads=args.num_query_groups or heads, head_dim=args.kv_channels or args.hidden_size // heads,
        ffn_hidden_size=args.ffn_hidden_size or 0, vocab_size=args.padded_vocab_size or args.vocab_size,
        rms_eps=args.norm_epsilon, rope_theta=float(args.rotary_base), qk_norm=bool(args.qk_layernorm),
        qkv_bias=bool(args.add_qkv_bias), tie_embeddings=not args.untie_embeddings_and_output_weights,
        num_experts=args.num_experts or 0, moe_top_k=args.moe_router_topk if moe else 0,
        moe_ffn_hidden_size=(args.moe_ffn_hidden_size or 0) if moe else 0,
        hf_architecture=(("Glm4MoeForCausalLM" if getattr(args, "moe_router_score_function", "softmax") == "sigmoid"
                          else "Qwen3MoeForCausalLM") if moe
                         else "Glm4ForCausalLM" if getattr(args, "post_self_attn_layernorm", False)
                         else "Qwen3ForCausalLM" if args.qk_layernorm else "Qwen2ForCausalLM" if args.add_qkv_bias else "LlamaForCausalLM"),
        post_norms=_sandwich_norms(args), rope_interleaved=bool(getattr(args, "rotary_interleaved", False)),
        # GLM-4.5 / DeepSeek-V3 style routing and shared experts (Megatron flag names)
        router_score=getattr(args, "moe_router_score_function", "softmax") if moe else "softmax",
        router_bias=bool(getattr(args, "moe_router_enable_expert_bias", False)) and moe,
        routed_scaling_factor=float(getattr(args, "moe_router_topk_scaling_factor", None) or 1.0),
        n_group=int(getattr(args, "moe_router_num_groups", None) or 1), topk_group=int(getattr(args, "moe_router_group_topk", None) or 1),
        shared_expert_ffn=int(getattr(args, "moe_shared_expert_intermediate_size", None) or 0) if moe else 0,
        shared_expert_gate=bool(getattr(args, "moe_shared_expert_gate", False)) and moe,
        first_dense_layers=_first_dense_layers(getattr(args, "moe_layer_freq", "1"), args.num_layers) if moe else 0,
        rotary_dim=(int(round((args.kv_channels or args.hidden_size // heads) * float(args.rotary_percent)))
                    if float(getattr(args, "rotary_percent", 1.0) or 1.0) != 1.0 else 0),
        # Megatron's --use-rope-scaling is the Llama-3.1 recipe with --rotary-scaling-factor (default 8)
        rope_scaling=({"rope_type": "llama3", "factor": float(args.rotary_scaling_factor or 8.0), "low_freq_factor": 1.0,
                       "high_freq_factor": 4.0, "original_max_position_embeddings": 8192}
                      if getattr(args, "use_rope_scaling", False) else None),
    )
