"""What happens to a flag that this framework parses but does not (yet) act on.

The command line mirrors the reference's (miles/utils/arguments.py:106-2589 plus the Megatron flags its launchers
pass), so that its launch scripts keep working. Every parsed flag falls in one of three classes:

* **consumed**: some module reads ``args.<dest>``;
* ``REJECT``: the flag changes the model, the numerics or the topology and the feature is not built. Setting
  it to anything but its default raises at start-up: a run never silently trains a different model;
* ``IGNORED``: the flag tunes a component that does not exist here (a Megatron / TransformerEngine kernel switch,
  a Ray placement hint, a Mooncake transport setting) or names the only behaviour this framework has. It is
  accepted; setting it to a non-default value logs one warning.

``tests/test_data_and_args.py`` walks the parser and fails when a flag is in none of the three classes, so a new flag
cannot be added without deciding what it does.
"""
from __future__ import annotations

import warnings

# dest -> why it cannot be honoured
REJECT = {
    # model architecture that is not built
    "apply_layernorm_1p": "zero-centred (1 + w) layer norm",
    "attention_output_gate": "gated attention output (Qwen3-Next style)",
    "attention_dropout": "dropout (post-training runs without it; only 0.0 is supported)",
    "hidden_dropout": "dropout (post-training runs without it; only 0.0 is supported)",
    "normalization": "normalisation other than RMSNorm",
    "position_embedding_type": "position embeddings other than rotary",
    "no_position_embedding": "models without rotary position embedding",
    "original_max_position_embeddings": "YaRN rope scaling",
    "beta_fast": "YaRN rope scaling",
    "beta_slow": "YaRN rope scaling",
    "mscale": "YaRN rope scaling",
    "mscale_all_dim": "YaRN rope scaling",
    "kv_lora_rank": "multi-latent attention",
    "q_lora_rank": "multi-latent attention",
    "qk_head_dim": "multi-latent attention",
    "qk_pos_emb_head_dim": "multi-latent attention",
    "v_head_dim": "multi-latent attention",
    "moe_router_pre_softmax": "softmax before the top-k over all experts is the only router order built",
    "moe_router_bias_update_rate": "updating the router's selection bias from the expert load (the bias is loaded and kept)",
    "moe_router_load_balancing_type": "router load-balancing losses",
    "moe_aux_loss_coeff": "router auxiliary loss",
    "moe_latent_size": "latent MoE",
    "moe_token_drop_policy": "token dropping (the dispatch here is dropless)",
    "enable_mtp_training": "multi-token-prediction layers",
    "multimodal_keys": "multimodal inputs",
    "freeze_indexer": "sparse-attention indexer models",
    # numerics that are not built
    "fp8_format": "FP8 / MXFP8 training GEMMs (block-scaled GEMMs serve the rollout only: --rollout-quantization)",
    "fp8_recipe": "FP8 / MXFP8 training GEMMs (block-scaled GEMMs serve the rollout only: --rollout-quantization)",
    "fp8_param_gather": "FP8 parameter all-gather",
    "fp4_format": "NVFP4 training GEMMs",
    "te_precision_config_file": "per-layer precision recipes",
    "num_layers_at_start_in_bf16": "per-layer precision recipes",
    "num_layers_at_end_in_bf16": "per-layer precision recipes",
    "extra_high_precision_layers_hf": "per-layer precision recipes",
    "extra_high_precision_layers_megatron": "per-layer precision recipes",
    "true_on_policy_mode": "bit-identical trainer / rollout numerics",
    "moe_router_dtype": "router precision other than fp32",
    # topology / backends that are not built
    "virtual_pipeline_model_parallel_size": "interleaved pipeline stages",
    "expert_tensor_parallel_size": "tensor parallelism inside experts",
    "qkv_format": "padded [batch, seq] batches (sequences are always packed)",
    "lora_type": "canonical LoRA",
    "experts_shared_outer_loras": "LoRA on experts",
    "multi_lora_backend_path": "pluggable multi-LoRA backends",
    "multi_lora_http_server_path": "pluggable multi-LoRA servers",
    "opd_topk_per_position": "per-position token lists in teacher scoring requests",
}

# dest -> why nothing needs to happen
IGNORED = {
    "dashboard_flush_interval": "dashboard events are appended to their files as they happen: there is no buffer to flush",
    "mtp_num_layers": "the multi-token-prediction layer is not built: the model trains and serves without it (training it, --enable-mtp-training, is rejected)",
    # sharded backend: activations are always recomputed per layer; checkpoints stage through host copies per unit
    "gradient_checkpointing": "layer inputs are the only activations kept: every layer is recomputed in the backward",
    "fsdp_state_dict_cpu_offload": "checkpoint and export copies are always staged in host memory, unit by unit",
    # Megatron / TransformerEngine kernel and fusion switches: one fused sm_100a path exists here
    "attention_backend": "one attention implementation (tcgen05 flash attention)",
    "attention_softmax_in_fp32": "softmax statistics are always fp32",
    "transformer_impl": "one implementation",
    "moe_grouped_gemm": "experts always run as grouped GEMMs",
    "moe_permute_fusion": "permutation is always fused",
    "moe_token_dispatcher_type": "one dispatcher (peer-memory all-to-all)",
    "moe_enable_deepep": "one dispatcher (peer-memory all-to-all)",
    "moe_router_padding_for_quantization": "no FP8 training path to pad for",
    "no_gradient_accumulation_fusion": "weight gradients always accumulate in the GEMM epilogue",
    "no_masked_softmax_fusion": "fused attention",
    "no_rope_fusion": "rope is always fused with the q/k norm",
    "disable_bias_linear": "projections have no bias unless the model config says so",
    "group_query_attention": "derived from the head counts",
    "use_rotary_position_embeddings": "rotary embedding is the only position embedding",
    "recompute_granularity": "activations are always recomputed layer by layer",
    "recompute_method": "activations are always recomputed layer by layer",
    "recompute_num_layers": "activations are always recomputed layer by layer",
    "recompute_loss_function": "the LM head runs in row chunks and recomputes its logits in the backward",
    "overlap_grad_reduce": "the partitioned optimizer reduces inside its own kernels",
    "overlap_param_gather": "the partitioned optimizer pushes parameters inside its own kernels",
    "overlap_cpu_optimizer_d2h_h2d": "host-resident optimizer state is always streamed on side streams",
    "use_distributed_post": "no Megatron post-processing step",
    "reuse_grad_buf_for_mxfp8_param_ag": "no FP8 parameter all-gather",
    "rematerialize_param_from_master_weight": "the bf16 weight is the upper half of the master: nothing to rematerialise",
    "check_rematerialize_param_from_master_weight": "the bf16 weight is the upper half of the master: nothing to rematerialise",
    "seq_length": "sequences are packed; the token cap per micro-batch is --max-tokens-per-gpu",
    "make_vocab_size_divisible_by": "the vocabulary is not padded",
    "tokenizer_model": "the tokenizer comes from --hf-checkpoint",
    "megatron_to_hf_mode": "one converter (native names <-> HF names)",
    "linear_attention_backend": "no linear-attention models",
    "dsa_attention_backend": "no sparse-attention models",
    "miles_dsa_topk_backend": "no sparse-attention models",
    "log_interval": "metrics are logged every rollout",
    # cluster plumbing of the reference (Ray, Mooncake, proxies)
    "num_gpus_per_node": "ranks come from torchrun",
    "critic_num_nodes": "the critic shares the actor's ranks",
    "critic_num_gpus_per_node": "the critic shares the actor's ranks",
    "pin_rollout_manager_to_head": "no Ray placement",
    "train_env_vars": "ranks inherit the launcher's environment",
    "train_memory_margin_bytes": "memory is planned by TrainActor (choose_memory_plan)",
    "mooncake_replica_num": "no Mooncake transport (weights move over NVLink / NCCL)",
    "mooncake_store_init_kwargs": "no Mooncake transport (weights move over NVLink / NCCL)",
    "p2p_transfer_num_workers": "no RDMA transfer workers",
    "p2p_transfer_timeout": "no RDMA transfer workers",
    "http_proxy": "engines are reached directly",
    "rollout_buffer_url": "no external rollout buffer service",
    "sglang_lora_use_virtual_experts": "the engine applies adapters as dense deltas",
    "lora_sync_from_tensor": "adapters always travel as tensors",
    "lora_base_cpu_backup": "base weights stay on the device",
    "memory_recorder": "one memory recorder (torch)",
    "wandb_always_use_train_step": "metrics are keyed by rollout id",
    "wandb_random_suffix": "run names are used as given",
    "custom_update_weight_post_write_path": "no weight files are written during an in-memory update",
    "update_weight_local_checkpoint_dir": "disk-delta updates write under --update-weight-disk-dir",
    "low_memory_resume": "resume loads one rank file at a time already",
    # batching / scheduling details of the reference's Ray pipeline
    "allow_partial_train_step": "trailing samples of a rollout always train as a smaller last step",
    "data_pad_size_multiplier": "packed micro-batches are not padded (the kernels take any token count)",
    "delay_split_train_data_by_dp": "a rank trains on the samples its own engine generated: there is no split to delay",
    "fetch_trajectory_retry_times": "the reference does not read it either",
    "min_batch_collection_ratio": "the reference does not read it either",
    "rollout_task_type": "the reference does not read it either",
    "dumper_source_patcher_config_inference": "the source patcher rewrites Megatron / SGLang sources, which do not exist here",
    "dumper_source_patcher_config_train": "the source patcher rewrites Megatron / SGLang sources, which do not exist here",
    "mtp_loss_scaling_factor": "the multi-token-prediction layer is not built, so its loss has no weight to scale",
    "opd_reward_weight_mode": "weights the per-token terms of multi-token (student-side top-k) distillation, which is not built",
}


def apply(args, defaults: dict) -> None:
    """Raise for a REJECT flag that is set; warn once for an IGNORED flag that is set. ``defaults``: dest -> parser default."""
    for dest, why in REJECT.items():
        if not hasattr(args, dest):
            continue
        v, d = getattr(args, dest), defaults.get(dest)
        if v == d or v in (None, False, [], {}, ""):
            continue
        if dest in ("attention_dropout", "hidden_dropout") and float(v) == 0.0:
            continue
        if dest == "rotary_percent" and float(v) == 1.0:
            continue
        if dest in ("moe_aux_loss_coeff", "moe_router_bias_update_rate") and float(v) == 0.0:
            continue
        if dest in ("num_layers_at_start_in_bf16", "num_layers_at_end_in_bf16") and int(v) == 0:
            continue
        if dest == "expert_tensor_parallel_size" and int(v) == 1:
            continue
        if dest == "moe_router_load_balancing_type" and float(getattr(args, "moe_aux_loss_coeff", 0.0) or 0.0) == 0.0:
            continue  # any balancing loss with coefficient zero is no loss at all
        if dest == "moe_router_pre_softmax":
            continue  # scores are always computed over all experts before the top-k (the order this flag asks for)
        raise NotImplementedError(f"--{dest.replace('_', '-')} {v!r}: {why} is not built in this framework; "
                                  "the flag is rejected rather than ignored")
    noted = []
    for dest, why in IGNORED.items():
        if not hasattr(args, dest):
            continue
        v, d = getattr(args, dest), defaults.get(dest)
        if isinstance(d, str) and not isinstance(v, str):  # argparse converts string defaults (JSON flags)
            try:
                import json

                d = json.loads(d)
            except ValueError:
                pass
        if v != d:
            noted.append(f"--{dest.replace('_', '-')} ({why})")
    if noted:
        warnings.warn("flags accepted for launch-script compatibility that change nothing here: " + "; ".join(noted), stacklevel=2)
