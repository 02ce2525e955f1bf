"""The trainer of one rank: the six-method backend contract ``init / train / update_weights / save_model /
sleep / wake_up`` (reference: miles/ray/train_actor.py:153-184 and the Megatron actor in
miles/backends/megatron_utils/actor.py:88-872), implemented natively on the flat parameter store.

One RL step (``train``): split the rollout over data-parallel ranks -> pack token-capped micro-batches
-> [reference-model log-probs] -> actor log-probs (the "old" policy, with routing recorded or replayed)
-> advantages / returns (+ whitening over DP) -> ``num_steps_per_rollout`` optimizer steps of
forward/backward over the micro-batches -> gradient reduction -> clip + fused Adam -> metrics.
"""
from __future__ import annotations

import math
import os
import time
from typing import Optional

import torch
import torch.distributed as dist

from ..models import ParamStore, build_model
from ..parallel.state import ParallelState, get_parallel_state
from ..rl.advantages import compute_advantages_and_returns
from ..rl.losses import LossConfig, SegmentReducer, policy_loss, sft_loss, value_loss
from ..utils.arguments import model_config_from_args
from ..utils.misc import load_function
from ..utils.timer import Timer
from .data import MicroBatch, build_micro_batches, split_by_dp
from .optimizer import FlatAdam, OptimConfig

_DT = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16}


EP_ENGINE_MIN_RANKS = 99  # expert-parallel groups of at least this many ranks serve the rollout expert parallel too


def replica_wanted(args, ep_size: int) -> bool:
    """Whether the colocated engine of an expert-parallel trainer serves from a full copy of the experts.
    ``--rollout-replicate-experts`` / ``--no-rollout-replicate-experts`` decide; by default small groups (two ranks)
    take the replica and larger ones the expert-parallel engine, which shares the expert weight stream."""
    v = getattr(args, "rollout_replicate_experts", None)
    if v is None:
        return ep_size < EP_ENGINE_MIN_RANKS
    return bool(v)


def choose_memory_plan(total_bytes: int, dense_params: int, expert_params: int, reserve_frac: float = 0.16,
                       extra_resident_bytes: int = 0, kv_bytes: int = 0, dp_size: int = 1, state: str = "fp32",
                       host_bytes: Optional[int] = None) -> dict:
    """Where the optimizer state of the expert group lives. The numerics do not depend on the placement:
    bf16 weights whose fp32 master is kept as (bf16 weight, signed 16-bit remainder), Adam moments in ``state``
    precision (fp32 like the reference's default optimizer, or bf16 like its precision-aware optimizer), fp32
    gradient accumulation for the replicated parameters and bf16 for the experts (that buffer shares its bytes with
    the KV cache of the colocated engine). Per expert parameter that is 2 B of weight on the device and 2 + 2 x
    moment-size bytes of optimizer state; the plan keeps the share of the state that fits next to everything else
    on the device and streams the rest through pinned host memory every optimizer step.

    ``reserve_frac`` of the device is left for activations, exchange buffers and the allocator;
    ``extra_resident_bytes`` is whatever else will stay resident (e.g. a full expert replica for the engine);
    ``kv_bytes`` the KV pool the engine will want (it shares the expert-gradient arena, so the larger of the two
    counts); the replicated parameters' state is partitioned over ``dp_size`` ranks; ``host_bytes`` is the pinned
    host memory this rank may take (None: unknown, not checked). Raises when device plus host cannot hold the state:
    nothing is silently degraded."""
    msize = 4 if state == "fp32" else 2
    bpp = 2 + 2 * msize
    state_bytes = expert_params * bpp
    dense = dense_params * (2 + 4) + dense_params * bpp // max(dp_size, 1)
    resident = dense + expert_params * 2 + max(int(kv_bytes), expert_params * 2) + int(extra_resident_bytes)
    room = int(total_bytes * (1.0 - reserve_frac)) - resident
    plan = dict(expert_grad="bf16", state=state, master=True, offload=False, resident_frac=1.0,
                name=f"fp32 master, {state} moments")
    if state_bytes > room:
        frac = max(0.0, min(1.0, room / max(state_bytes, 1)))
        frac = int(frac * 64) / 64.0  # whole chunks, rounded down
        on_host = int(state_bytes * (1 - frac))
        if host_bytes is not None and on_host > host_bytes:
            raise MemoryError(
                f"optimizer state of {state_bytes / 1e9:.0f} GB ({bpp} B per expert parameter, {state} moments): "
                f"{state_bytes * frac / 1e9:.0f} GB fit on the device, the remaining {on_host / 1e9:.0f} GB exceed the "
                f"{host_bytes / 1e9:.0f} GB of host memory this rank may pin. Use more GPUs"
                + (", or --use-precision-aware-optimizer --exp-avg-dtype bf16 --exp-avg-sq-dtype bf16" if state == "fp32" else ""))
        plan.update(offload=True, resident_frac=frac, name=plan["name"] + ", %d%% of the expert state streamed from host" % round(100 * (1 - frac)))
    return plan


def host_memory_per_rank(local_world: int) -> Optional[int]:
    """Pinned host bytes one rank may take: 80 % of what is available now (the cgroup limit if that is lower),
    divided among the ranks of this node. None when it cannot be read."""
    try:
        import psutil

        avail = psutil.virtual_memory().available
    except Exception:
        return None
    try:
        txt = open("/sys/fs/cgroup/memory.max").read().strip()
        if txt.isdigit():
            cur = int(open("/sys/fs/cgroup/memory.current").read().strip())
            avail = min(avail, int(txt) - cur)
    except Exception:
        pass
    return int(avail * 0.8) // max(local_world, 1)


def wanted_kv_bytes(args, cfg, n_rep: int) -> int:
    """The KV pool a colocated engine asks for: every running request at the full context length."""
    local_batch = max(1, (args.rollout_batch_size * args.n_samples_per_prompt + n_rep - 1) // n_rep)
    max_running = getattr(args, "sglang_max_running_requests", None) or min(512, max(local_batch, 1))
    max_ctx = getattr(args, "rollout_max_context_len", None) or ((getattr(args, "rollout_max_prompt_len", None) or 1024)
                                                                  + args.rollout_max_response_len + 8)
    page = getattr(args, "engine_page_size", 64)
    per_tok = 2 * cfg.num_layers * cfg.num_kv_heads * cfg.head_dim * 2
    return int(max_running * (max_ctx + page) * per_tok)


class TrainActor:
    def __init__(self, args, role: str = "actor", ps: Optional[ParallelState] = None, store: Optional[ParamStore] = None):
        self.args = args
        self.role = role
        self.ps = ps or get_parallel_state()
        if getattr(args, "custom_megatron_init_path", None):
            # a user hook that runs once per trainer process after the parallel groups exist and before the model is
            # built (the reference calls it at the end of its Megatron initialisation): fn(args)
            load_function(args.custom_megatron_init_path)(args)
        self.cfg = model_config_from_args(args)
        self.device = self.ps.device
        self.on_gpu = self.device.type == "cuda"
        backend = getattr(args, "model_backend", "auto")
        want_b200 = backend == "b200" or (backend == "auto" and self.on_gpu and self.cfg.head_dim == 128)
        self.dtype = torch.bfloat16 if want_b200 else (torch.float32 if not self.on_gpu else torch.bfloat16)
        ep = self.ps.ep.size if self.cfg.is_moe else 1
        tp = self.ps.tp.size
        # --train-backend fsdp: pure data parallelism with parameters, master weights and moments sharded per unit
        # over the data-parallel ranks (miles_b200/fsdp)
        self.fsdp = getattr(args, "train_backend", "megatron") == "fsdp"
        if self.fsdp and store is None:
            from ..fsdp import FsdpParamStore, build_mesh

            if tp > 1 or self.ps.pp.size > 1 or self.ps.ep.size > 1:
                raise ValueError("--train-backend fsdp is data parallel only (optionally with context parallelism): "
                                 "tensor / pipeline / expert parallel sizes must be 1")
            if getattr(args, "lora_rank", 0):
                raise NotImplementedError("--lora-rank with --train-backend fsdp is not built")
            self.mesh = build_mesh(self.ps, int(getattr(args, "dp_replicate_size", 1) or 1))
            store = FsdpParamStore(self.cfg, self.device, self.dtype, self.mesh, init_std=getattr(args, "init_std", 0.02),
                                   seed=args.seed, num_buffers=int(getattr(args, "fsdp_num_unit_buffers", 2) or 2))
        if store is None:
            store = ParamStore(self.cfg, self.device, self.dtype, ep_size=ep, ep_rank=self.ps.ep.rank if ep > 1 else 0,
                               init_std=getattr(args, "init_std", 0.02), seed=args.seed, tp_size=tp, tp_rank=self.ps.tp.rank,
                               pp_size=self.ps.pp.size, pp_rank=self.ps.pp.rank,
                               pp_first_layers=getattr(args, "decoder_first_pipeline_num_layers", None),
                               pp_last_layers=getattr(args, "decoder_last_pipeline_num_layers", None))
        self.store = store
        self.pipe = None
        if self.ps.pp.size > 1:
            from ..parallel.pipeline_parallel import PipeGroup, PipelineSchedule

            self.pipe = PipelineSchedule(PipeGroup(self.ps.pp.group, self.ps.pp.rank, self.ps.pp.size, self.ps.pp.ranks), self.device)
        self.tp_exchange = None
        if tp > 1:
            from ..parallel.tensor_parallel import TensorParallel

            assert want_b200, "tensor parallelism needs the sm_100a model path"
            max_tok = max(getattr(args, "max_tokens_per_gpu", None) or 0, getattr(args, "engine_max_prefill_tokens", 16384), 4096)
            from ..parallel.topology import peer_memory_ok

            # peer-memory kernels need every rank of the group on this node; a group across nodes reduces with NCCL
            self.tp_exchange = TensorParallel(self.ps.tp.group, self.ps.tp.rank, tp, self.device, self.cfg.hidden_size, max_tok,
                                              fused=peer_memory_ok(self.ps.tp.group, tp, getattr(args, "fused_comm", True)))
        self.ep_dispatcher = None
        if ep > 1:
            from ..parallel.expert_parallel import ExpertParallel

            max_tok = max(getattr(args, "max_tokens_per_gpu", None) or 0, getattr(args, "engine_max_prefill_tokens", 16384),
                          (getattr(args, "rollout_max_context_len", None) or 0), 4096)
            from ..parallel.topology import peer_memory_ok

            self.ep_dispatcher = ExpertParallel(self.cfg, self.ps, max_tokens=max_tok,
                                                fused=peer_memory_ok(self.ps.ep.group, ep, getattr(args, "fused_comm", True)))
        provider = getattr(args, "custom_model_provider_path", None)
        if provider:
            # a plug-in builds the model (see miles_b200/plugins): it says itself whether it runs under autograd
            self.model = load_function(provider)(args=args, cfg=self.cfg, store=store, ep=self.ep_dispatcher, tp=self.tp_exchange,
                                                 role=role)
            self.is_torch = bool(getattr(self.model, "uses_autograd", not want_b200))
        else:
            self.model = build_model(self.cfg, store, "b200" if want_b200 else "torch", ep=self.ep_dispatcher, tp=self.tp_exchange)
            self.is_torch = not want_b200
        self.loss_cfg = LossConfig.from_args(args)
        self.loss_cfg.args = args  # plug-ins (custom TIS / reducer functions) read their own options from the command line
        if getattr(args, "custom_tis_function_path", None):
            self.loss_cfg.custom_tis_fn = load_function(args.custom_tis_function_path)
        if getattr(args, "custom_pg_loss_reducer_function_path", None):
            self.loss_cfg.custom_pg_reducer_fn = load_function(args.custom_pg_loss_reducer_function_path)
        self.custom_loss_fn = load_function(args.custom_loss_function_path) if getattr(args, "custom_loss_function_path", None) else None
        self.opt: Optional[FlatAdam] = None
        self.plan: dict = {}
        self.arena: Optional[torch.Tensor] = None  # see lend_arena()
        self.weights_backup: dict = {}   # tag -> pinned host copies of the flat buffers (ref / old_actor / teacher)
        self.rollout_engines: list = []
        self.global_step = 0
        self.loaded_rollout_id: Optional[int] = None
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self._value_head = None
        self.cell_group = None  # ft.indep_dp.ReconfigurableGroup when this trainer is one cell of several
        # audit trail (--enable-witness / --save-debug-event-data): every trained sample id is counted through the same
        # commit / discard boundary as the optimizer step, and steps are logged with a weight checksum
        self.witness = None
        self.events = None
        if getattr(args, "enable_witness", False) or getattr(args, "save_debug_event_data", None) or getattr(args, "enable_event_analyzer", False):
            from ..utils.audit import EventLogger, Witness

            self.events = EventLogger(getattr(args, "save_debug_event_data", None), role, self.ps.rank)
            if getattr(args, "enable_witness", False):
                self.witness = Witness(int(getattr(args, "witness_buffer_size", 1 << 20) or (1 << 20)))
        self.dumper = None
        if getattr(args, "dumper_enable", False):
            from ..utils.dumper import Dumper

            self.dumper = Dumper(getattr(args, "dumper_dir", None) or "/tmp/dumper", self.ps.rank)
            # a phase is dumped when its flag is given, or when none of the three is (dump everything)
            chosen = {"inference": getattr(args, "dumper_inference", None), "fwd_only": getattr(args, "dumper_fwd_only", None),
                      "fwd_bwd": getattr(args, "dumper_fwd_bwd", None)}
            self.dumper.phases = {k for k, v in chosen.items() if v} or set(chosen)
        if getattr(args, "deterministic_mode", False):
            # reproducible kernels where a choice exists: torch ops, cuBLAS workspaces, fixed-order gradient reductions
            # (the attention backward still accumulates dQ with atomics, the one order-dependent sum of this trainer)
            os.environ.setdefault("CUBLAS_WORKSPACE_CONFIG", ":4096:8")
            os.environ.setdefault("NCCL_ALGO", "Ring")
            torch.use_deterministic_algorithms(True, warn_only=True)
            args.debug_deterministic_collective = True
        if role == "critic":
            self._init_value_head()
        self._setup_optimizer()
        self.lora = None
        if getattr(args, "lora_rank", 0) and args.lora_rank > 0 and role == "actor":
            from ..lora import LoRAManager

            self.lora = LoRAManager(self.store, args.lora_rank, args.lora_alpha or args.lora_rank, args.target_modules or "all-linear",
                                    lr=args.lr, weight_decay=args.weight_decay, seed=args.seed, betas=(args.adam_beta1, args.adam_beta2),
                                    tp_group=self.ps.tp.group if self.ps.tp.size > 1 else None)
            self.opt = None  # base weights are frozen: only the adapters have optimizer state
            if getattr(args, "lora_adapter_path", None):
                self.lora.load(args.lora_adapter_path)
        if getattr(args, "load", None):
            from ..checkpoint import load_checkpoint

            # the rollout id the checkpoint was written after (None: weights only, start from rollout 0);
            # load_checkpoint restores global_step (optimizer steps) itself
            self.loaded_rollout_id = load_checkpoint(self, args.load, getattr(args, "ckpt_step", None))
            if getattr(args, "reset_optimizer_states", False) and self.opt is not None:
                self.opt.reset_state()  # keep the weights (and their fp32 master), restart the moments and the schedule
        if getattr(args, "use_opd", False) and getattr(args, "opd_type", None) == "megatron" and role == "actor" \
                and getattr(args, "opd_teacher_load", None):
            # on-policy distillation against a teacher the trainer itself evaluates: its weights live in a pinned host
            # copy and are swapped in for one log-prob pass per rollout (--opd-teacher-load / --opd-teacher-ckpt-step)
            from ..checkpoint import load_weights_into_backup

            self.backup_weights("teacher")
            load_weights_into_backup(self, "teacher", args.opd_teacher_load, getattr(args, "opd_teacher_ckpt_step", None))
        need_ref = (args.kl_coef != 0 or args.use_kl_loss) and role == "actor"
        if need_ref:
            self.backup_weights("ref")
            if getattr(args, "ref_load", None) and args.ref_load != getattr(args, "load", None):
                from ..checkpoint import load_weights_into_backup

                load_weights_into_backup(self, "ref", args.ref_load, getattr(args, "ref_ckpt_step", None))

    # ------------------------------------------------------------------ setup
    def _init_value_head(self) -> None:
        g = torch.Generator(device="cpu").manual_seed(self.args.seed + 17)
        w = torch.empty(1, self.cfg.hidden_size).normal_(0, 0.02, generator=g)
        self._value_head = w.to(self.device, torch.float32).requires_grad_(True)

    def _setup_optimizer(self) -> None:
        a = self.args
        if getattr(a, "debug_disable_optimizer", False):
            return
        dense = self.store.sizes["dense"]
        expert = self.store.sizes["expert"]
        if self.on_gpu:
            total = torch.cuda.get_device_properties(self.device).total_memory
            extra = 0
            colocated = self.role == "actor" and not getattr(a, "debug_train_only", False) and not getattr(a, "rollout_engine_urls", None)
            if self.fsdp and colocated:
                # the colocated engine holds a whole copy of the model next to this rank's shards, plus the unit buffers
                extra = sum(self.store.full_sizes.values()) * 2 + sum(self.store.max_padded.values()) * 12
            elif (self.cfg.is_moe and self.ps.ep.size > 1 and colocated and self.ps.tp.size == 1
                    and replica_wanted(a, self.ps.ep.size)):
                # the colocated engine will hold all experts in a buffer of its own (see RLLoop._build_engine; this
                # rank's share is stored twice: the trainer's flat shard and its slice of every replica tensor)
                extra = expert * self.ps.ep.size * 2
            kv = 0
            if colocated:
                kv = min(wanted_kv_bytes(a, self.cfg, self.ps.dp_cp.size * self.ps.pp.size),
                         int(total * float(getattr(a, "sglang_mem_fraction_static", 0.7))))
            # moments: fp32 unless the precision-aware optimizer flags ask for 16 bits
            state = "fp32"
            if getattr(a, "use_precision_aware_optimizer", False) or a.exp_avg_dtype != "fp32" or a.exp_avg_sq_dtype != "fp32":
                state = a.exp_avg_dtype if a.exp_avg_dtype in ("bf16", "fp32") else "bf16"
            local_world = int(os.environ.get("LOCAL_WORLD_SIZE", self.ps.world_size))
            plan = choose_memory_plan(total, dense, expert, extra_resident_bytes=extra, kv_bytes=kv, dp_size=self.ps.dp_cp.size,
                                      state=state, host_bytes=host_memory_per_rank(local_world))
        else:
            plan = dict(expert_grad="fp32", state="fp32", master=False, offload=False, resident_frac=1.0, name="cpu")
        if getattr(a, "main_params_dtype", "fp32") != "fp32":
            plan["master"] = False
            plan["name"] += ", no fp32 master"
        if self.fsdp and getattr(a, "fsdp_cpu_offload", False):
            plan["offload"], plan["resident_frac"] = True, 0.0
            if not self.store.sizes.get("expert"):
                import warnings

                # host-resident optimizer state is built for the expert group (where the bulk of a MoE model's state
                # lives and one weight-decay value covers the whole buffer); a dense model's shards stay on the device
                warnings.warn("--fsdp-cpu-offload: this model has no expert parameters, its optimizer state shards stay on the device")
        if getattr(a, "optimizer_cpu_offload", False) or getattr(a, "offload_optimizer_states", False):
            plan["offload"], plan["resident_frac"] = True, 0.0
        if getattr(a, "accumulate_allreduce_grads_in_fp32", False) and self.on_gpu and self.cfg.is_moe:
            # fp32 accumulation for the experts too, when twice the bytes still fit beside the rest
            total = torch.cuda.get_device_properties(self.device).total_memory
            if expert * 4 + expert * 2 + dense * 6 + (expert * 10 if not plan["offload"] else 0) < 0.7 * total:
                plan["expert_grad"] = "fp32"
        if self.store.dtype == torch.float32:
            plan["master"] = False
        self.plan = plan
        self._expert_grad_dtype = torch.bfloat16 if (plan["expert_grad"] == "bf16" and self.store.dtype == torch.bfloat16) else torch.float32
        self.store.allocate_grads(torch.float32, self._expert_grad_dtype)
        warmup = a.lr_warmup_iters or 0
        if getattr(a, "lr_warmup_fraction", None) and (a.lr_decay_iters or 0) > 0:
            warmup = int(a.lr_warmup_fraction * a.lr_decay_iters)  # Megatron: a fraction of the decay horizon
        if self.role == "critic" and getattr(a, "critic_lr_warmup_iters", 0):
            warmup = a.critic_lr_warmup_iters
        oc = OptimConfig(lr=a.lr if self.role == "actor" else (a.critic_lr or a.lr), beta1=a.adam_beta1, beta2=a.adam_beta2,
                         eps=a.adam_eps, weight_decay=a.weight_decay, clip_grad=a.clip_grad, state_dtype=_DT[plan["state"]],
                         master_weights=plan["master"], offload_states=plan["offload"],
                         offload_resident_frac=plan.get("resident_frac", 0.0) if plan["offload"] else 0.0,
                         lr_decay_style=a.lr_decay_style,
                         lr_warmup_iters=warmup, lr_decay_iters=a.lr_decay_iters or 0, min_lr=a.min_lr,
                         skip_nonfinite=not getattr(a, "no_check_for_nan_in_loss_and_grad", False),
                         lr_wsd_decay_iters=a.lr_wsd_decay_iters or 0)
        if self.fsdp:
            if getattr(a, "stream_optimizer_state_to_disk", False) or getattr(a, "optimizer", "adam") != "adam":
                raise NotImplementedError("--train-backend fsdp steps with Adam on the resident or host-offloaded shards")
            if not getattr(a, "keep_fp32_master", True):
                oc.master_weights = False
            self.dense_shard = None
            # gradients arrive reduced over the shard group; every rank's slice counts once in the global norm
            self.opt = FlatAdam(self.store, oc, shard_group=self.store.group)
            return
        if getattr(a, "stream_optimizer_state_to_disk", False) or getattr(a, "offload_train_target", "cpu") == "disk":
            # optimizer state in files on a local disk, streamed through the device bucket by bucket
            # (--stream-optimizer-state-to-disk, or --offload-train-target disk): for models whose state fits neither
            # in device nor in host memory
            from .nvme_optimizer import NvmeStreamedAdam

            d = getattr(a, "offload_train_disk_dir", None) or os.path.join(getattr(a, "save", None) or "/tmp", "optimizer_stream")
            mdt = getattr(a, "stream_optimizer_state_moment_dtype", "fp32")
            assert mdt in ("fp32", "bf16", "fp16"), "--stream-optimizer-state-moment-dtype: fp8 moments are not built"
            self.dense_shard = None
            self.opt = NvmeStreamedAdam(self.store, os.path.join(d, f"rank_{self.ps.rank:05d}"), lr=oc.lr,
                                        betas=(oc.beta1, oc.beta2), eps=oc.eps, weight_decay=oc.weight_decay,
                                        bucket_elems=max(1, int(getattr(a, "offload_train_disk_chunk_mb", 256)) * (1 << 20) // 4),
                                        moment_dtype=mdt, clip_grad=oc.clip_grad)
            return
        if getattr(a, "optimizer", "adam") == "muon":
            from .muon import Muon, MuonConfig

            self.dense_shard = None
            self.opt = Muon(self.store, oc, MuonConfig(momentum=getattr(a, "muon_momentum", 0.95), nesterov=not getattr(a, "muon_no_nesterov", False),
                                                       ns_steps=getattr(a, "muon_num_ns_steps", 5), scale_mode=getattr(a, "muon_scale_mode", "spectral"),
                                                       extra_scale=getattr(a, "muon_extra_scale_factor", 1.0),
                                                       split_qkv=not getattr(a, "muon_no_split_qkv", False)),
                            ep_group=self.ps.ep.group, tp_group=self.ps.tp.group if self.ps.tp.size > 1 else None,
                            pp_group=self.ps.pp.group if self.ps.pp.size > 1 else None)
            return
        dense_shard = None
        if (self.on_gpu and self.ps.dp_cp.size > 1 and self.ps.tp.size == 1 and self.store.dtype == torch.bfloat16
                and getattr(a, "fused_comm", True) and getattr(a, "use_distributed_optimizer", True) and self.ps.dp_cp.size <= 8
                and self._dp_on_one_node()):
            from ..parallel.dp_optimizer import ShardedDenseAdam

            # replicated parameters: reduce-scatter + Adam on the owned range + all-gather as peer-memory kernels
            dense_shard = ShardedDenseAdam(self.store, self.ps.dp_cp.group, self.ps.dp_cp.rank, self.ps.dp_cp.size, self.device, oc)
        self.dense_shard = dense_shard
        self.opt = FlatAdam(self.store, oc, dp_group=self.ps.dp_cp.group, ep_group=self.ps.ep.group,
                            tp_group=self.ps.tp.group if self.ps.tp.size > 1 else None, dense_shard=dense_shard,
                            pp_group=self.ps.pp.group if self.ps.pp.size > 1 else None)

    def _dp_on_one_node(self) -> bool:
        from ..parallel.topology import group_is_single_node

        return group_is_single_node(self.ps.dp_cp.group, self.ps.dp_cp.size)

    # ------------------------------------------------------------------ weight tags (ref / old_actor / teacher)
    def backup_weights(self, tag: str) -> None:
        """Pinned-host copy of the live weights under ``tag`` (reference: miles/utils/tensor_backper.py:22-180)."""
        bk = self.weights_backup.get(tag)
        if bk is None:
            bk = {g: torch.empty(t.shape, dtype=t.dtype, pin_memory=self.on_gpu) for g, t in self.store.flat.items()}
            self.weights_backup[tag] = bk
        for g, t in self.store.flat.items():
            bk[g].copy_(t, non_blocking=True)
        if self.on_gpu:
            torch.cuda.current_stream().synchronize()

    def restore_weights(self, tag: str) -> None:
        for g, t in self.store.flat.items():
            t.copy_(self.weights_backup[tag][g], non_blocking=True)

    class _Swapped:
        def __init__(self, actor, tag):
            self.a, self.tag = actor, tag

        def __enter__(self):
            self.a.backup_weights("_live")
            self.a.restore_weights(self.tag)

        def __exit__(self, *exc):
            self.a.restore_weights("_live")

    def with_weights(self, tag: str):
        return TrainActor._Swapped(self, tag)

    # ------------------------------------------------------------------ forward passes
    def _set_cp(self, mb: MicroBatch) -> None:
        """Tell the model how the micro-batch is cut along the sequence (context parallelism)."""
        cp = mb.extras.get("cp")
        if cp is None:
            if hasattr(self.model, "cp_ctx"):
                self.model.cp_ctx = None
            return
        if not self.is_torch and self.cfg.num_kv_heads % cp[1] != 0:
            raise NotImplementedError(f"context parallelism on the sm_100a path trades sequence shards for head shards: the "
                                      f"{self.cfg.num_kv_heads} key / value heads must divide by the context-parallel size {cp[1]}")
        self.model.cp_ctx = (cp[0], cp[1], cp[2], self.ps.cp.group, getattr(self.ps, "cp_comm_type", "p2p"), cp[3])

    def _forward_logprobs(self, mb: MicroBatch, replay=None, record=None):
        inv_t = 1.0 / self.args.rollout_temperature
        self._set_cp(mb)
        chunk = getattr(self.args, "log_probs_chunk_size", -1) or -1
        if chunk > 0 and hasattr(self.model, "lm_chunk"):
            self.model.lm_chunk = int(chunk)  # rows of the LM head (logits -> log-prob / entropy) computed at a time
        if self.is_torch:
            return self.model.forward_logprobs(mb.tokens, mb.positions, mb.cu_seqlens, mb.rows, mb.targets, inv_t,
                                               replay=replay, record=record)
        return self.model.forward_logprobs(mb.tokens, mb.positions, mb.cu_seqlens, mb.rows, mb.targets, inv_t,
                                           replay=replay, record=record, max_seqlen=mb.max_seqlen)

    def _replay_for(self, mb: MicroBatch, phase: str):
        a = self.args
        if not self.cfg.is_moe:
            return None
        if a.use_rollout_routing_replay and mb.replay is not None:
            return mb.replay
        if a.use_routing_replay and phase == "train":
            return mb.extras.get("recorded_routing")
        return None

    @torch.no_grad()
    def compute_log_probs(self, mbs: list, key: str = "log_probs", with_entropy: bool = False) -> None:
        if self.pipe is not None:
            return self._compute_log_probs_pipelined(mbs, key, with_entropy)
        for mb in mbs:
            record = [] if (self.cfg.is_moe and self.args.use_routing_replay and not self.args.use_rollout_routing_replay
                            and key == "log_probs") else None
            lp, ent = self._forward_logprobs(mb, self._replay_for(mb, "logprob"), record)
            if self.dumper is not None and "fwd_only" in self.dumper.phases:
                self.dumper.configure("fwd_only", self.global_step)
                self.dumper.dump(f"{key}_mb{mbs.index(mb)}", lp, samples=mb.sample_indices)
            mb.extras[key] = lp
            if with_entropy:
                mb.extras["entropy"] = ent
            if record:
                mb.extras["recorded_routing"] = torch.stack(record, 1)

    # ------------------------------------------------------------------ pipeline parallel passes
    def _act_meta(self, mbs: list):
        H = self.cfg.hidden_size
        return lambda i: ((mbs[i].tokens.shape[0], H), self.store.dtype)

    @torch.no_grad()
    def _compute_log_probs_pipelined(self, mbs: list, key: str, with_entropy: bool) -> None:
        """Forward-only pipeline; the last stage's log-probs (and entropies, recorded routing) are then shared with
        the other stages so that every stage runs the same advantage / bookkeeping code."""
        a, pp, cfg = self.args, self.ps.pp, self.cfg
        inv_t = 1.0 / a.rollout_temperature
        want_record = cfg.is_moe and a.use_routing_replay and not a.use_rollout_routing_replay and key == "log_probs"
        records: dict = {}
        results: dict = {}

        def fwd(i, x_in):
            mb = mbs[i]
            self._set_cp(mb)
            rec = [] if want_record else None
            records[i] = rec
            replay = self._replay_for(mb, "logprob")
            if self.store.is_last_stage:
                results[i] = self.model.forward_logprobs(mb.tokens, mb.positions, mb.cu_seqlens, mb.rows, mb.targets, inv_t,
                                                         replay=replay, record=rec, max_seqlen=mb.max_seqlen, x_in=x_in)
                return None
            kw = {} if self.is_torch else {"max_seqlen": mb.max_seqlen}
            return self.model.forward_hidden(mb.tokens, mb.positions, mb.cu_seqlens, replay=replay, record=rec, x_in=x_in, **kw)

        self.pipe.run_forward_only(len(mbs), self._act_meta(mbs), fwd)
        src = pp.ranks[-1]
        lo = self.store.layer_range[0]
        moe_before = sum(cfg.layer_is_moe(j) for j in range(lo))
        n_moe = sum(cfg.layer_is_moe(j) for j in range(cfg.num_layers))
        for i, mb in enumerate(mbs):
            n = mb.targets.shape[0]
            buf = torch.stack(results[i][:2]) if self.store.is_last_stage else torch.empty(2, n, dtype=torch.float32, device=self.device)
            dist.broadcast(buf, src=src, group=pp.group)
            mb.extras[key] = buf[0].contiguous()
            if with_entropy:
                mb.extras["entropy"] = buf[1].contiguous()
            if want_record:
                full = torch.zeros(mb.tokens.shape[0], n_moe, cfg.moe_top_k, dtype=torch.int32, device=self.device)
                if records[i]:
                    full[:, moe_before:moe_before + len(records[i])] = torch.stack(records[i], 1).to(torch.int32)
                dist.all_reduce(full, group=pp.group)  # stages hold disjoint layers: the sum is the concatenation
                mb.extras["recorded_routing"] = full

    def _forward_backward_pipelined(self, chunk: list, scale: float, metrics_acc: dict) -> None:
        """1F1B over the micro-batches of one optimizer step. Intermediate stages keep the per-layer inputs of their
        in-flight micro-batches (at most `stages after this one + 1`); the last stage runs forward, loss and backward
        of a micro-batch back to back."""
        inv_t = 1.0 / self.args.rollout_temperature
        saved: dict = {}
        last = self.store.is_last_stage
        if self.is_torch:
            return self._forward_backward_pipelined_autograd(chunk, scale, metrics_acc)

        def fwd(i, x_in):
            mb = chunk[i]
            if last:
                saved[i] = x_in
                return None
            inputs: list = []
            y = self.model.forward_hidden(mb.tokens, mb.positions, mb.cu_seqlens, replay=self._replay_for(mb, "train"),
                                          max_seqlen=mb.max_seqlen, save_inputs=inputs, x_in=x_in)
            inputs.pop()  # the stage output itself
            saved[i] = inputs
            return y

        def bwd(i, dy):
            mb = chunk[i]
            replay = self._replay_for(mb, "train")
            if last:
                _, m, _, _ = self.model.forward_backward(mb.tokens, mb.positions, mb.cu_seqlens, mb.rows, mb.targets, inv_t,
                                                         self._loss_closure(mb, scale), replay=replay, max_seqlen=mb.max_seqlen,
                                                         x_in=saved.pop(i))
                for k, v in m.items():
                    metrics_acc[k] = metrics_acc.get(k, 0.0) + v.detach().float() * scale
                return self.model.last_dx_in
            return self.model.layers_backward(saved.pop(i), dy, mb.tokens, mb.positions, mb.cu_seqlens, mb.max_seqlen, replay)

        self.pipe.run_1f1b(len(chunk), self._act_meta(chunk), fwd, bwd)
        if self.cfg.tie_embeddings and (self.store.is_first_stage or last):
            pass  # reduced in _reduce_grads (all stages take part in the collective)

    def _forward_backward_pipelined_autograd(self, chunk: list, scale: float, metrics_acc: dict) -> None:
        """The same schedule for the PyTorch model: a stage keeps the autograd graph of its in-flight micro-batches
        and back-propagates the gradient it receives (the last stage: its loss)."""
        inv_t = 1.0 / self.args.rollout_temperature
        saved: dict = {}
        last, first = self.store.is_last_stage, self.store.is_first_stage
        model = self.model
        model.set_requires_grad(True)

        def fwd(i, x_in):
            mb = chunk[i]
            self._set_cp(mb)
            leaf = None if first else x_in.detach().requires_grad_(True)
            if last:
                saved[i] = leaf
                return None
            with torch.enable_grad():
                y = model.forward_hidden(mb.tokens, mb.positions, mb.cu_seqlens, replay=self._replay_for(mb, "train"), x_in=leaf)
            saved[i] = (leaf, y)
            return y.detach()

        def bwd(i, dy):
            mb = chunk[i]
            self._set_cp(mb)
            if last:
                leaf = saved.pop(i)
                lp, ent = model.forward_logprobs(mb.tokens, mb.positions, mb.cu_seqlens, mb.rows, mb.targets, inv_t,
                                                 replay=self._replay_for(mb, "train"), with_grad=True, x_in=leaf)
                loss, m = self._loss_closure(mb, scale)(lp, ent)
                loss.backward()
                for k, v in m.items():
                    metrics_acc[k] = metrics_acc.get(k, 0.0) + v.detach().float() * scale
            else:
                leaf, y = saved.pop(i)
                y.backward(dy)
            model.accumulate_autograd_grads()
            return None if leaf is None else leaf.grad

        self.pipe.run_1f1b(len(chunk), self._act_meta(chunk), fwd, bwd)
        model.set_requires_grad(False)

    # ------------------------------------------------------------------ the RL step
    def _stage(self, data: dict) -> list:
        a = self.args
        if getattr(self, "_local_data", False):
            ids = list(range(len(data["tokens"])))  # the caller already holds exactly this rank's share
        else:
            # the ranks of one context-parallel group work on the same samples (each on its share of the tokens)
            ids = split_by_dp(data, self.ps.dp.size, balance=getattr(a, "balance_data", False))[self.ps.dp.rank]
        lens = [len(data["tokens"][i]) for i in ids]
        n_mb = None
        moe_layers = sum(self.cfg.layer_is_moe(i) for i in range(self.cfg.num_layers))
        kw = dict(pin=self.on_gpu, num_moe_layers=moe_layers, top_k=self.cfg.moe_top_k, sample_ids=ids)
        if a.use_dynamic_batch_size:
            from .data import num_micro_batches_for

            n_mb = num_micro_batches_for(lens, a.max_tokens_per_gpu) if lens else 0
            if self.ps.world_size > 1:
                t = torch.tensor([n_mb], dtype=torch.int64, device=self.device)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                n_mb = int(t.item())
            if getattr(a, "balance_by_flops", False):
                # partition by estimated FLOPs (linear + quadratic attention term) instead of token counts: sequences of
                # very different lengths then cost the micro-batches about the same time
                kw["weights"] = "flops"
            if self.ps.world_size > 1 or getattr(a, "balance_by_flops", False):
                mbs = build_micro_batches(data, num_micro_batches=max(n_mb, 1), **kw)
            else:
                mbs = build_micro_batches(data, max_tokens_per_gpu=a.max_tokens_per_gpu, **kw)
        else:
            mbs = build_micro_batches(data, micro_batch_size=a.micro_batch_size, **kw)
        out = []
        cp = self.ps.cp.size
        if cp > 1:
            assert a.advantage_estimator in ("grpo", "reinforce_plus_plus_baseline") or a.loss_type == "sft_loss", \
                "context parallelism supports estimators whose per-token terms need no other rank's tokens"
        for mb in mbs:
            d = mb.cp_shard(cp, self.ps.cp.rank, "allgather" if getattr(a, "allgather_cp", False) else "zigzag").to_device(self.device)
            self.h2d_bytes += d.h2d_bytes
            out.append(d)
        return out

    def _advantages(self, mbs: list) -> None:
        a = self.args
        if getattr(a, "disable_compute_advantages_and_returns", False):
            return
        for mb in mbs:
            adv, ret, kl = compute_advantages_and_returns(
                advantage_estimator=a.advantage_estimator, rewards=mb.rewards, cu=mb.resp_cu, loss_mask=mb.loss_mask,
                log_probs=mb.extras.get("log_probs") if not a.use_rollout_logprobs else mb.rollout_log_probs,
                ref_log_probs=mb.extras.get("ref_log_probs"), values=mb.extras.get("values"),
                teacher_log_probs=mb.teacher_log_probs if a.use_opd else None, kl_coef=a.kl_coef, kl_loss_type=a.kl_loss_type,
                gamma=a.gamma, lambd=a.lambd, normalize_advantages=False, opd_kl_coef=a.opd_kl_coef if a.use_opd else 0.0)
            mb.extras["advantages"], mb.extras["returns"], mb.extras["kl"] = adv, ret, kl
        if a.normalize_advantages and mbs:
            from ..rl.advantages import whiten

            allv = torch.cat([mb.extras["advantages"] for mb in mbs])
            allm = torch.cat([mb.loss_mask for mb in mbs])
            w = whiten(allv, allm, self.ps.dp_cp.group, reduce=self.ps.dp_cp.size > 1)
            off = 0
            for mb in mbs:
                n = mb.loss_mask.numel()
                mb.extras["advantages"] = w[off:off + n]
                off += n

    def _loss_closure(self, mb: MicroBatch, scale: float):
        a, lc = self.args, self.loss_cfg
        reducer = SegmentReducer(mb.seg, mb.loss_mask, mb.denoms, per_token=a.calculate_per_token_loss, num_samples=mb.num_samples)

        def fn(lp, ent):
            if a.loss_type == "sft_loss":
                loss, m = sft_loss(lc, lp, reducer=reducer)
            elif a.loss_type == "custom_loss":
                loss, m = self.custom_loss_fn(a, mb, lp, ent, reducer)
            else:
                loss, m = policy_loss(lc, lp, ent, old_log_probs=mb.extras.get("log_probs"), advantages=mb.extras["advantages"],
                                      reducer=reducer, rollout_log_probs=mb.rollout_log_probs,
                                      ref_log_probs=mb.extras.get("ref_log_probs"))
            return loss * scale, m

        return fn

    def train(self, rollout_id: int, data: dict) -> dict:
        a = self.args
        T = Timer()
        t_start = time.perf_counter()
        dump = getattr(a, "save_debug_train_data", None)
        if dump:
            # per-step training inputs of this rank, for replay with --load-debug-rollout-data style tooling
            path = dump.format(rollout_id=rollout_id, rank=self.ps.rank)
            os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
            torch.save({"rollout_id": rollout_id, "rank": self.ps.rank,
                        "data": {k: v for k, v in data.items() if isinstance(v, (list, tuple, int, float, str, torch.Tensor))}}, path)
        with T.context("data_preprocess"):
            mbs = self._stage(data)
        n_tokens_local = sum(mb.num_tokens for mb in mbs)
        self._last_seq_lens = [int(x) for mb in mbs for x in (mb.cu_seqlens[1:] - mb.cu_seqlens[:-1]).tolist()]
        need_old = not (a.use_rollout_logprobs or a.skip_actor_forward_only) or a.use_routing_replay and not a.use_rollout_routing_replay
        if a.loss_type == "sft_loss":
            need_old = False
        if "ref" in self.weights_backup and a.loss_type == "policy_loss":
            with T.context("ref_log_probs"), self.with_weights("ref"):
                self.compute_log_probs(mbs, "ref_log_probs")
        if "teacher" in self.weights_backup and a.loss_type == "policy_loss":
            with T.context("teacher_log_probs"), self.with_weights("teacher"):
                self.compute_log_probs(mbs, "teacher_log_probs")
            for mb in mbs:
                mb.teacher_log_probs = mb.extras["teacher_log_probs"]
        for k in ("train_log_probs", "train_fwd_bwd", "train_optimizer"):
            T.reset(k)
        if getattr(a, "custom_megatron_before_log_prob_hook_path", None):
            # reference signature: hook(args, model, store_prefix)
            load_function(a.custom_megatron_before_log_prob_hook_path)(a, self.model, "")
        if need_old:
            with T.context("log_probs"), T.cuda_span("train_log_probs"):
                self.compute_log_probs(mbs, "log_probs", with_entropy=getattr(a, "use_rollout_entropy", False))
        if a.loss_type == "policy_loss":
            if data.get("values") is not None:
                for mb in mbs:
                    mb.extras["values"] = torch.cat([torch.as_tensor(data["values"][i], dtype=torch.float32)
                                                     for i in mb.sample_indices]).to(self.device)
            self._advantages(mbs)
        metrics_acc: dict = {}
        grad_norm = torch.zeros((), device=self.device)
        wid_of: dict = {}
        if self.witness is not None:
            # a slot of the witness ring for every sample this rank trains in this rollout (the same slots again when a
            # failed attempt of the rollout is retried)
            from ..utils.audit import ev_witness_allocate

            sids = sorted({int(i) for mb in mbs for i in mb.sample_indices})
            wids, stale = self.witness.allocate(rollout_id, sids)
            wid_of = dict(zip(sids, wids))
            if self.events is not None:
                self.events.log(ev_witness_allocate(rollout_id, sids, wids, stale))
        with T.context("actor_train"):
            steps = a.num_steps_per_rollout or 1
            per_step = max(1, math.ceil(len(mbs) / steps))
            gbs = a.global_batch_size or max(1, len(data["tokens"]))
            for s in range(steps):
                chunk = mbs[s * per_step:(s + 1) * per_step]
                if not chunk:
                    continue
                self.store.zero_grads()
                if getattr(a, "custom_megatron_before_train_step_hook_path", None):
                    # reference signature: hook(args, rollout_id, step_id, model, optimizer, opt_param_scheduler)
                    load_function(a.custom_megatron_before_train_step_hook_path)(a, rollout_id, s, self.model, self.opt, None)
                if a.calculate_per_token_loss:
                    tok = torch.stack([mb.loss_mask.sum() for mb in chunk]).sum()
                    if self.ps.dp_cp.size > 1:  # a size-1 axis has no group object, and None would mean the whole world
                        dist.all_reduce(tok, group=self.ps.dp_cp.group)
                    scale = 1.0 / max(float(tok.item()), 1.0)
                else:
                    scale = 1.0 / gbs
                with T.cuda_span("train_fwd_bwd"):
                    if self.pipe is not None:
                        self._forward_backward_pipelined(chunk, scale, metrics_acc)
                    else:
                        for mb in chunk:
                            m = self._forward_backward(mb, scale)
                            for k, v in m.items():
                                metrics_acc[k] = metrics_acc.get(k, 0.0) + v.detach().float() * scale
                    self._reduce_grads()
                    if getattr(self, "cell_group", None) is not None:
                        from ..ft.indep_dp import cross_cell_grad_sync

                        # independent data-parallel cells: average over the cells, and apply the step only if every
                        # cell got through it (a discarded step leaves weights and optimizer state untouched)
                        if not cross_cell_grad_sync(self, self.cell_group):
                            self.discarded_steps = getattr(self, "discarded_steps", 0) + 1
                            self.store.zero_grads()
                            if self.witness is not None:
                                self.witness.discard()
                            if self.events is not None:
                                from ..utils.audit import ev_train_step

                                ids = [i for mb in chunk for i in mb.sample_indices]
                                self.events.log(ev_train_step(rollout_id, self.global_step, len(ids), "discarded", ids))
                            continue
                if self.witness is not None:
                    self.witness.touch(wid_of[i] for mb in chunk for i in mb.sample_indices)
                with T.cuda_span("train_optimizer"):
                    if self.lora is not None:
                        self.lora.grads_from_weight_grads()
                        grad_norm = self.lora.step(a.clip_grad)
                    elif self.opt is not None:
                        grad_norm = self.opt.step(1.0)
                if getattr(a, "ci_test", False):
                    from ..utils.ci_checks import check_grad_norm

                    check_grad_norm(a, float(grad_norm), rollout_id, s, self.role, self.ps.rank)
                self.global_step += 1
                if self.witness is not None:
                    self.witness.commit()
                if self.events is not None:
                    from ..utils.audit import ev_train_step, ev_weight_checksum, ev_witness_snapshot

                    ids = [i for mb in chunk for i in mb.sample_indices]
                    self.events.log(ev_train_step(rollout_id, self.global_step, len(ids), "normal", ids))
                    if self.witness is not None:
                        # what the table holds for this step's samples now (read back, not assumed)
                        self.events.log(ev_witness_snapshot(rollout_id, self.global_step, self.witness.counts(wid_of[i] for i in ids)))
                    if getattr(a, "enable_event_analyzer", False):
                        ck = self.store.checksum()
                        self.events.log(ev_weight_checksum(self.global_step, self.store.version, f"{ck.get('dense', 0.0):.6e}"))
        if self.on_gpu:
            torch.cuda.synchronize()
        elapsed = time.perf_counter() - t_start
        T.flush_cuda()
        out = self._finalize_metrics(metrics_acc, grad_norm, n_tokens_local, elapsed, len(mbs))
        for k in ("train_log_probs", "train_fwd_bwd", "train_optimizer"):
            out[f"perf/{k}_time"] = float(T.log_dict().get(k, 0.0))
        if getattr(a, "ci_test", False) and (a.num_steps_per_rollout or 1) == 1 and not a.use_rollout_logprobs:
            from ..utils.ci_checks import check_first_step_kl

            # one optimizer step per rollout: the whole rollout was trained with the weights that computed its log-probs
            check_first_step_kl(a, out, 0, self.global_step - 1)
        if getattr(a, "keep_old_actor", False):
            self.backup_weights("old_actor")
        if a.ref_update_interval and "ref" in self.weights_backup and (rollout_id + 1) % a.ref_update_interval == 0:
            self.backup_weights("ref")
        return out

    def _forward_backward(self, mb: MicroBatch, scale: float) -> dict:
        inv_t = 1.0 / self.args.rollout_temperature
        fn = self._loss_closure(mb, scale)
        replay = self._replay_for(mb, "train")
        self._set_cp(mb)
        if self.is_torch:
            self.model.set_requires_grad(True)
            lp, ent = self.model.forward_logprobs(mb.tokens, mb.positions, mb.cu_seqlens, mb.rows, mb.targets, inv_t,
                                                  replay=replay, with_grad=True)
            loss, m = fn(lp, ent)
            loss.backward()
            self.model.accumulate_autograd_grads()
            self.model.set_requires_grad(False)
            return m
        _, m, lp, _ = self.model.forward_backward(mb.tokens, mb.positions, mb.cu_seqlens, mb.rows, mb.targets, inv_t, fn,
                                                  replay=replay, max_seqlen=mb.max_seqlen)
        if self.dumper is not None and "fwd_bwd" in self.dumper.phases:
            self.dumper.configure("fwd_bwd", self.global_step)
            self.dumper.dump(f"log_probs_s{mb.sample_indices[0]}", lp, samples=mb.sample_indices)
        return m

    def _reduce_grads(self) -> None:
        """Sum dense gradients over dp x cp and expert gradients over the experts' own data-parallel group."""
        if self.fsdp:
            # each unit was reduce-scattered as the backward left it: flush the last one (and sum over replicas)
            self.store.finish_grads()
            return
        if self.ps.world_size <= 1:
            return
        if self.ps.tp.size > 1:
            # q/k norm weights are shared by all heads: each tensor-parallel rank holds the sum over its own heads
            names = [n for n in self.store.grads if n.endswith(("attn.q_norm.weight", "attn.k_norm.weight"))]
            if names:
                buf = torch.stack([self.store.grads[n].float() for n in names])
                dist.all_reduce(buf, group=self.ps.tp.group)
                for n, row in zip(names, buf):
                    self.store.grads[n].copy_(row)
        if self.ps.pp.size > 1 and self.cfg.tie_embeddings:
            # the first stage's embedding and the last stage's LM head are one parameter: both need the summed gradient
            H = self.cfg.hidden_size
            ge = self.store.grads.get("embed.weight")
            buf = ge.float() if ge is not None else torch.zeros(self.cfg.vocab_size, H, dtype=torch.float32, device=self.device)
            dist.all_reduce(buf, group=self.ps.pp.group)
            if ge is not None:
                ge.copy_(buf)
        g = self.store.grad
        reduce = dist.all_reduce
        if getattr(self.args, "debug_deterministic_collective", False):
            # gather + fixed-order tree sum instead of the library's ring / tree of the day (--debug-deterministic-collective)
            from ..utils.det_collectives import det_all_reduce

            reduce = det_all_reduce
        if self.ps.dp_cp.size > 1 and g["dense"] is not None and g["dense"].numel() and getattr(self, "dense_shard", None) is None:
            reduce(g["dense"], group=self.ps.dp_cp.group)  # with the partitioned optimizer the step itself reduces
        if self.ps.expert_dp.size > 1 and g["expert"] is not None and g["expert"].numel():
            reduce(g["expert"], group=self.ps.expert_dp.group)

    def _finalize_metrics(self, acc: dict, grad_norm, n_tokens_local: int, elapsed: float, n_mb: int) -> dict:
        keys = sorted(acc)
        vals = torch.stack([acc[k].reshape(()) for k in keys]) if keys else torch.zeros(0, device=self.device)
        extra = torch.tensor([float(n_tokens_local)], device=self.device)
        if self.ps.world_size > 1:
            if keys and self.ps.dp_cp.size > 1:
                dist.all_reduce(vals, group=self.ps.dp_cp.group)
            dist.all_reduce(extra)
            extra = extra / (self.ps.tp.size * self.ps.pp.size)  # ranks of one replica staged the same tokens
        out = {f"train/{k}": float(v) for k, v in zip(keys, vals.tolist())}
        if self.ps.pp.size > 1:
            # only the last stage computes the loss: every stage reports its metrics
            box = [out]
            dist.broadcast_object_list(box, src=self.ps.pp.ranks[-1], group=self.ps.pp.group)
            out = dict(box[0])
        out["train/grad_norm"] = float(grad_norm)
        if self.opt is not None:
            from .optimizer import lr_at

            out["train/lr"] = lr_at(self.opt.cfg, max(self.opt.step_count - 1, 0))
        out["train/step"] = self.global_step
        out["perf/actor_train_time"] = elapsed
        out["perf/actor_train_tok_per_s"] = float(extra[0]) / max(elapsed, 1e-9)
        lens = getattr(self, "_last_seq_lens", None)
        if lens and elapsed > 0:
            from ..utils.metric_utils import perf_metrics

            # per-GPU TFLOP/s and MFU of this rank's share (reference: miles/utils/train_metric_utils.py:36-48)
            pm = perf_metrics(self.cfg, lens, elapsed, 1, peak_tflops=getattr(self.args, "mfu_peak_tflops", None))
            out.update({k: v for k, v in pm.items() if k != "perf/actor_train_tok_per_s"})
        out["perf/num_micro_batches"] = n_mb
        return out

    # ------------------------------------------------------------------ critic (PPO)
    @torch.no_grad()
    def compute_values(self, mbs: list) -> None:
        for mb in mbs:
            h = self.model.forward_hidden(mb.tokens, mb.positions, mb.cu_seqlens) if self.is_torch else \
                self.model.forward_hidden(mb.tokens, mb.positions, mb.cu_seqlens, max_seqlen=mb.max_seqlen)
            mb.extras["values"] = (h[mb.rows].float() @ self._value_head.t())[:, 0]

    def train_critic(self, rollout_id: int, data: dict) -> dict:
        """Critic step of shared actor/critic PPO: values -> GAE returns -> clipped value loss.
        The values computed before the update are written back into ``data['values']`` for the actor."""
        a = self.args
        mbs = self._stage(data)
        self.compute_values(mbs)
        for mb in mbs:
            adv, ret, _ = compute_advantages_and_returns(
                advantage_estimator="ppo", rewards=mb.rewards, cu=mb.resp_cu, loss_mask=mb.loss_mask, values=mb.extras["values"],
                kl_coef=0.0, gamma=a.gamma, lambd=a.lambd)
            mb.extras["returns"] = ret
        gbs = a.global_batch_size or max(1, len(data["tokens"]))
        self.store.zero_grads()
        if self._value_head.grad is not None:
            self._value_head.grad = None
        acc: dict = {}
        for mb in mbs:
            reducer = SegmentReducer(mb.seg, mb.loss_mask, mb.denoms, per_token=a.calculate_per_token_loss, num_samples=mb.num_samples)
            old_v, ret = mb.extras["values"], mb.extras["returns"]

            def head(hr, old_v=old_v, ret=ret, reducer=reducer):
                v = (hr @ self._value_head.t())[:, 0]
                loss, m = value_loss(self.loss_cfg, v, old_values=old_v, returns=ret, reducer=reducer)
                return loss / gbs, m

            if self.is_torch:
                self.model.set_requires_grad(True)
                with torch.enable_grad():
                    h = self.model.forward_hidden(mb.tokens, mb.positions, mb.cu_seqlens)
                    loss, m = head(h[mb.rows].float())
                    loss.backward()
                self.model.accumulate_autograd_grads()
                self.model.set_requires_grad(False)
            else:
                _, m = self.model.forward_backward_hidden(mb.tokens, mb.positions, mb.cu_seqlens, mb.rows, head, max_seqlen=mb.max_seqlen)
            for k, v in m.items():
                acc[k] = acc.get(k, 0.0) + v.detach().float() / gbs
        self._reduce_grads()
        if self.ps.dp_cp.size > 1 and self._value_head.grad is not None:
            dist.all_reduce(self._value_head.grad, group=self.ps.dp_cp.group)
        gn = self.opt.step(1.0) if self.opt is not None else torch.zeros(())
        with torch.no_grad():
            if self._value_head.grad is not None:
                self._value_head -= (a.critic_lr or a.lr) * self._value_head.grad
                self._value_head.grad = None
        self.global_step += 1
        # hand the pre-update values to the actor in sample order
        vals = [None] * len(data["tokens"])
        for mb in mbs:
            cu = mb.resp_cu.tolist()
            v = mb.extras["values"].detach().cpu()
            for j, i in enumerate(mb.sample_indices):
                vals[i] = v[cu[j]:cu[j + 1]].tolist()
        data["values"] = vals
        out = self._finalize_metrics(acc, gn, sum(mb.num_tokens for mb in mbs), 0.0, len(mbs))
        return {k: v for k, v in out.items() if k.startswith("train/")}

    # ------------------------------------------------------------------ weight update, offload, checkpoints
    def connect_rollout_engines(self, engines: list) -> None:
        self.rollout_engines = list(engines)

    def update_weights(self) -> dict:
        from ..weight_sync import sync_weights

        with Timer().context("update_weights"):
            return sync_weights(self, self.rollout_engines)

    def lend_arena(self, min_bytes: int) -> torch.Tensor:
        """One device buffer that holds the expert gradients while training and is lent to the colocated
        engine (KV cache) while rolling out. The two uses never overlap in the synchronous loop, the
        addresses stay fixed (captured decode graphs remain valid), and nothing is freed or reallocated
        between phases. Returns the uint8 buffer (at least ``min_bytes`` long)."""
        if self.fsdp:
            # sharded gradients are small and the unit buffers come and go with sleep / wake: the arena is the cache's own
            if self.arena is None or self.arena.numel() < int(min_bytes):
                self.arena = None
                self.arena = torch.empty(max(int(min_bytes), 256), dtype=torch.uint8, device=self.device)
            return self.arena
        n = self.store.sizes.get("expert", 0) * torch.empty((), dtype=self._expert_grad_dtype).element_size()
        size = max(int(min_bytes), n, 256)
        if self.arena is None or self.arena.numel() < size:
            self.store.free_grads()
            self.arena = None
            if self.on_gpu:
                torch.cuda.empty_cache()
            self.arena = torch.empty(size, dtype=torch.uint8, device=self.device)
            self.store.allocate_grads(torch.float32, self._expert_grad_dtype, expert_storage=self.arena)
        return self.arena

    def sleep(self) -> None:
        """Release trainer-only device memory (gradients) so that the rollout engine can use it. With a lent
        arena the gradients already share their bytes with the KV cache and nothing has to move."""
        with Timer().context("sleep"):
            if self.fsdp:
                self.store.release_buffers()  # the full-unit buffers; the gradient shards stay
                if self.on_gpu:
                    torch.cuda.empty_cache()
                return
            if self.arena is not None:
                return
            self.store.free_grads()
            if self.on_gpu:
                torch.cuda.empty_cache()

    def wake_up(self) -> None:
        with Timer().context("wake_up"):
            if not self.store.grads:
                self.store.allocate_grads(torch.float32, getattr(self, "_expert_grad_dtype", torch.float32),
                                          expert_storage=self.arena)

    def save_model(self, rollout_id: int, force_sync: bool = False) -> None:
        from ..checkpoint import save_checkpoint

        with Timer().context("save_model"):
            if getattr(self.args, "save", None):
                d = save_checkpoint(self, self.args.save, rollout_id)
                if self.lora is not None and (self.ps.rank == 0 or (self.ps.tp.size > 1 and 0 in self.ps.tp.ranks)):
                    # the ranks of rank 0's tensor-parallel group gather the adapter together; rank 0 writes it
                    self.lora.save(os.path.join(d, "adapter"), getattr(self.args, "hf_checkpoint", None) or "",
                                   write_adapter=self.ps.rank == 0)
            if getattr(self.args, "save_hf", None):
                from ..checkpoint import export_hf

                export_hf(self, self.args.save_hf.format(rollout_id=rollout_id))
