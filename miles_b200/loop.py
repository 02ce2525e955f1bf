"""The synchronous RL loop of one rank (SPMD: one process per GPU, trainer and engine colocated).

Per rollout step (reference driver: train.py:22-150)::

    generate -> [offload rollout: free KV] -> [critic.train] -> actor.train -> save
             -> [offload train: free gradients] -> onload KV -> update_weights -> eval

Every rank owns a slice of the prompt stream and generates its own groups with its in-process engine;
the samples a rank generated are the samples it trains on, so no rollout data crosses GPUs (the
reference ships them through the Ray object store).  Collectives appear only inside the model (expert
parallel dispatch), in the gradient reduction and in metric aggregation.
"""
from __future__ import annotations

import asyncio
import copy
import os
import time
from typing import Optional

import torch
import torch.distributed as dist

from .engine import Engine
from .engine.client import EngineClient
from .parallel.state import ParallelState, init_parallel_state
from .rollout.base_types import RolloutFnConstructorInput, RolloutFnEvalInput, RolloutFnTrainInput
from .rollout.train_data import (compute_rollout_metrics, convert_samples_to_train_data, flatten_groups,
                                 postprocess_rollout_data)
from .trainer.actor import TrainActor
from .utils.misc import load_function, should_run_periodic_action
from .utils.timer import Timer


def _load_tokenizer(args):
    path = getattr(args, "hf_checkpoint", None)
    if not path or not os.path.isdir(path):
        return None
    try:
        from transformers import AutoTokenizer

        return AutoTokenizer.from_pretrained(path, trust_remote_code=True)
    except Exception:
        return None


class RLLoop:
    def __init__(self, args, ps: Optional[ParallelState] = None):
        self.args = args
        self.ps = ps or init_parallel_state(
            tp=args.tensor_model_parallel_size, pp=args.pipeline_model_parallel_size, cp=args.context_parallel_size,
            ep=args.expert_model_parallel_size, backend=None if args.distributed_backend == "nccl" else args.distributed_backend,
            timeout_minutes=args.distributed_timeout_minutes, cp_comm_type=getattr(args, "cp_comm_type", "p2p"))
        # ranks of one tensor-parallel group are one data-parallel replica: same seeds, same prompts, same samples
        # the stages of a pipeline each run their own engine on a full copy of the model and pool their samples
        # before training, so they count as rollout replicas too
        self.n_rep = self.ps.dp_cp.size * self.ps.pp.size
        self.rep = self.ps.dp_cp.rank * self.ps.pp.size + self.ps.pp.rank
        torch.manual_seed(args.seed + self.rep)
        self.tokenizer = _load_tokenizer(args)
        if self.ps.rank == 0 and os.environ.get("MILES_B200_ENV_REPORT", "1") != "0":
            # library versions, GPUs, collective-steering environment and git state as one marked JSON line in the log
            from .utils.env_report import collect_and_print

            try:
                collect_and_print()
            except Exception as e:  # noqa: BLE001  (a report must never stop a run)
                print(f"[miles_b200] environment report failed: {e!r}", flush=True)
        self.actor = TrainActor(args, "actor", self.ps)
        if self.ps.rank == 0 and os.environ.get("MILES_B200_ENV_REPORT", "1") != "0":
            # which clauses of the trainer / rollout numerical contract this configuration keeps: says where a
            # train / rollout log-prob difference may come from before the first step shows one
            from .true_on_policy import check, explain

            print(explain(check(args, self.actor.cfg)), flush=True)
        self.critic = None
        if getattr(args, "use_critic", False):
            cargs = copy.copy(args)
            cargs.load = getattr(args, "critic_load", None)
            cargs.kl_coef, cargs.use_kl_loss = 0.0, False
            self.critic = TrainActor(cargs, "critic", self.ps)
        self.engine: Optional[Engine] = None
        self.client: Optional[EngineClient] = None
        self.weight_updater = None
        self.fleet = None
        if getattr(args, "launch_rollout_fleet", False) and not getattr(args, "debug_train_only", False):
            args.rollout_engine_urls = self._launch_fleet()
        if getattr(args, "rollout_engine_urls", None) and not getattr(args, "debug_train_only", False):
            self._connect_remote_engines([u for u in args.rollout_engine_urls.split(",") if u])
        elif not getattr(args, "debug_train_only", False):
            if args.offload_train:
                self.actor.sleep()  # gradients are only needed inside train(); the KV cache gets the memory first
            self._build_engine()
        self.data_source = self._build_data_source()
        self.rollout_fn = self._build_rollout_fn()
        self.start_rollout_id = self._resume()
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        from .utils.ci_checks import metric_checker_from_args

        self.metric_checker = metric_checker_from_args(args)
        self.session_urls: list = []
        if getattr(args, "use_session_server", False) and self.ps.rank == 0:
            self.session_urls = self._start_session_servers()
            args.session_server_urls = self.session_urls  # generate functions hand these to their agent frameworks
        self.ft = None
        if getattr(args, "use_fault_tolerance", False):
            from .ft.runtime import FTRuntime

            self.ft = FTRuntime(self, args)
        self.tracker = None
        try:
            from .utils.tracking import init_tracking

            self.tracker = init_tracking(args, primary=self.ps.rank == 0)
        except Exception:
            self.tracker = None

    # ------------------------------------------------------------------ construction
    def _build_engine(self) -> None:
        a = self.args
        cfg = self.actor.cfg
        local_batch = max(1, (a.rollout_batch_size * a.n_samples_per_prompt + self.n_rep - 1) // self.n_rep)
        max_running = getattr(a, "sglang_max_running_requests", None) or min(512, max(local_batch, 1))
        max_ctx = getattr(a, "rollout_max_context_len", None) or ((getattr(a, "rollout_max_prompt_len", None) or 1024)
                                                                   + a.rollout_max_response_len + 8)
        page = getattr(a, "engine_page_size", 64)
        kv_bytes = None
        if self.actor.on_gpu:
            total = torch.cuda.get_device_properties(self.actor.device).total_memory
            frac = float(getattr(a, "sglang_mem_fraction_static", 0.7))
            budget = int(total * frac) - self.actor.store.nbytes()
            if getattr(self.actor, "fsdp", False):
                budget -= sum(self.actor.store.full_sizes.values()) * 2  # the engine's own whole copy of the model
            per_tok = 2 * cfg.num_layers * cfg.num_kv_heads * cfg.head_dim * 2
            want = max_running * (max_ctx + page) * per_tok
            # what is really free once weights, gradients and resident optimizer states are placed, keeping
            # a seventh of the device for activations; expert gradients count as free (the arena is shared)
            free_now = torch.cuda.mem_get_info(self.actor.device)[0]
            lend = 0
            if getattr(a, "share_kv_grad_memory", True) and self.actor.store.grad.get("expert") is not None:
                g = self.actor.store.grad["expert"]
                lend = g.numel() * g.element_size()
            room = free_now + lend - total // 7
            kv_bytes = max(min(budget, want, room), per_tok * page * 4)
        pipelined = self.ps.pp.size > 1
        sharded = getattr(self.actor, "fsdp", False)
        replicate = not pipelined and self.actor.ep_dispatcher is not None and self._replicate_experts_fits(kv_bytes)
        if replicate:
            # the worst case (every sequence at the full context length) almost never happens and the engine retracts
            # requests when the pool runs dry: with the replica resident, size the pool for 65 % of that worst case
            kv_bytes = max(min(kv_bytes, room - self._replica_bytes(), int(0.65 * want)), per_tok * page * 4)
        if pipelined or sharded:
            assert self.actor.ep_dispatcher is None and self.ps.tp.size == 1, \
                "the colocated engine of a pipelined or sharded trainer is built for tp = ep = 1"
            from .models import build_specs

            full_bytes = sum(sp.numel for sp in build_specs(cfg)) * 2
            if kv_bytes is not None:
                kv_bytes = max(min(kv_bytes, room - full_bytes), per_tok * page * 4)
        kv_storage = None
        if self.actor.on_gpu and getattr(a, "share_kv_grad_memory", True) and not getattr(a, "debug_rollout_only", False):
            # rollout and training alternate in this loop: the KV cache borrows the bytes of the expert gradients
            kv_storage = self.actor.lend_arena(kv_bytes)
        sync = ep_decode = None
        engine_model = self.actor.model
        self.rollout_store = None
        self.weight_pusher = None
        if replicate:
            # Rollout on a full replica of the experts: decode is bound by the weights it streams, not by capacity,
            # and a B200 holds all experts of this model many times over. Every rank then generates independently
            # with the single-GPU kernels (no dispatch / return per layer, no lockstep dummy steps); training stays
            # expert parallel, and the weight update all-gathers the updated expert shares into the replica.
            from .models import ParamStore, build_model

            ep = self.ps.ep
            from .parallel.topology import peer_memory_ok

            if (peer_memory_ok(ep.group, ep.size, getattr(a, "fused_comm", True)) and self.actor.store.dtype == torch.bfloat16
                    and ep.size <= 8 and getattr(a, "update_weight_transfer_mode", "broadcast") != "broadcast-nccl"):
                # the replica's experts live in a peer-mapped region: every rank stores its updated expert shard
                # straight into all replicas with one kernel (csrc/weight_push.cu) instead of an all-gather per tensor
                from .weight_sync.p2p_push import Layout, PushTarget, WeightPusher

                target = PushTarget.create(cfg, ep.group, ep.rank, ep.size, self.actor.device, groups=("expert",),
                                           share_dense=self.actor.store)
                self.rollout_store = target.store
                self.weight_pusher = WeightPusher(cfg, self.actor.store, target, ep.rank,
                                                  [Layout(ep_size=ep.size, ep_rank=r) for r in range(ep.size)],
                                                  [Layout() for _ in range(ep.size)], skip_groups=("dense",), amax_group=ep.group)
                self.rollout_store.weight_pusher = self.weight_pusher
            else:
                self.rollout_store = ParamStore(cfg, self.actor.device, self.actor.store.dtype, ep_size=1, init=False,
                                                share_dense=self.actor.store)
            engine_model = build_model(cfg, self.rollout_store, "b200")
        elif sharded:
            # the trainer holds one slice of every unit: the engine decodes on a whole copy that the weight update fills
            # with one all-gather per unit, straight into its flat buffers (miles_b200/fsdp/store.py)
            from .fsdp.store import FsdpWeightGather
            from .models import ParamStore, build_model

            self.rollout_store = ParamStore(cfg, self.actor.device, self.actor.store.dtype, init=False)
            self.rollout_store.weight_pusher = FsdpWeightGather(self.actor.store, self.rollout_store)
            engine_model = build_model(cfg, self.rollout_store, "b200" if not self.actor.is_torch else "torch")
        elif pipelined:
            # the trainer's stage holds part of the layers; the engine decodes on a copy of the whole model that the
            # weight update fills stage by stage (broadcasts inside the pipeline group)
            from .models import ParamStore, build_model

            self.rollout_store = ParamStore(cfg, self.actor.device, self.actor.store.dtype, init=False)
            engine_model = build_model(cfg, self.rollout_store, "b200" if not self.actor.is_torch else "torch")
        elif self.actor.ep_dispatcher is not None:
            from .engine.core import LockstepSync
            from .parallel.expert_parallel import ExpertParallel

            sync = LockstepSync(self.ps.gloo_world if self.ps.backend != "gloo" else None)
            from .parallel.topology import peer_memory_ok

            one_node = peer_memory_ok(self.ps.ep.group, self.ps.ep.size, getattr(a, "fused_comm", True))
            if self.actor.on_gpu and one_node and max_running <= 256 and not self.actor.is_torch:
                # decode steps: gather / partial-sum exchange with in-kernel flags (csrc/ep_decode.cu)
                from .parallel.ep_decode import EpDecodeLL

                ep_decode = EpDecodeLL(cfg, self.ps, max_rows=max(max_running, 8))
            else:
                ep_decode = ExpertParallel(cfg, self.ps, fused=one_node, max_tokens=max(max_running, 16))
        quant = getattr(a, "rollout_quantization", "none")
        if quant != "none" and self.actor.on_gpu and not self.actor.is_torch:
            if engine_model is self.actor.model:
                # the trainer keeps multiplying bf16 weights: the engine gets a model object of its own on the same store
                from .models import build_model

                engine_model = build_model(cfg, self.actor.store, "b200", ep=self.actor.ep_dispatcher, tp=self.actor.tp_exchange)
            engine_model.enable_block_scaled(quant)
        self.engine = Engine(engine_model, sync=sync, ep_decode=ep_decode, max_running=max_running, page_size=page, max_seq_len=max_ctx,
                             max_prefill_tokens=getattr(a, "engine_max_prefill_tokens", 16384), kv_mem_bytes=kv_bytes,
                             use_cuda_graph=not getattr(a, "sglang_disable_cuda_graph", False) and self.actor.on_gpu,
                             eos_token_id=getattr(self.tokenizer, "eos_token_id", None), kv_storage=kv_storage,
                             # prefix (radix) cache: on unless --sglang-disable-radix-cache, as in the reference's engines;
                             # lockstep expert-parallel engines keep it off (their ranks must run the same iterations)
                             prefix_cache=not getattr(a, "sglang_disable_radix_cache", False) and sync is None,
                             # a KV cache of its own that --offload-rollout releases: tagged virtual memory keeps the
                             # addresses (captured graphs stay valid across release / resume)
                             memory_saver=kv_storage is None and bool(getattr(a, "offload_rollout", False)))
        self.engine.seed_salt = int(getattr(a, "seed", 1234)) * 1000003 + self.ps.rank
        if sync is not None:
            self.engine.warm_up_decode_graphs()  # lockstep ranks capture their decode graphs together
        self.client = EngineClient([self.engine], self.tokenizer)
        self.actor.connect_rollout_engines([self.engine])
        if self.actor.on_gpu and self.actor.opt is not None and self.actor.plan.get("offload"):
            # everything resident is allocated now: whatever is left beyond the activation reserve takes moments back
            # from host memory (less to stream per optimizer step)
            free_now, total = torch.cuda.mem_get_info(self.actor.device)
            spare = free_now - total // 5
            t = torch.tensor([float(max(spare, 0))], device=self.actor.device)
            if self.ps.world_size > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MIN)
            self.actor.opt.promote_offloaded(int(t.item()))

    def _launch_fleet(self) -> str:
        """Start the rollout engines this job asks for (``--sglang-config`` file, or ``--rollout-num-gpus`` /
        ``--rollout-num-gpus-per-engine``) on the GPUs after the trainer's, from the first rank; every rank learns the
        URLs. The engines stop with the job."""
        import atexit

        a = self.args
        box = [None]
        if self.ps.rank == 0:
            from .engine.deployment import Deployment
            from .engine.fleet import Fleet

            dep = Deployment.from_yaml(a.sglang_config) if getattr(a, "sglang_config", None) else Deployment.from_args(a)
            dep.resolve(a)
            dev = getattr(a, "rollout_fleet_device", None)
            self.fleet = Fleet(dep, model_preset=getattr(a, "model_preset", None), base_port=a.rollout_fleet_base_port, device=dev,
                               first_gpu=0 if (dev or "").startswith("cpu") else self.ps.world_size).start()
            atexit.register(self.fleet.stop)
            box[0] = ",".join(self.fleet.updatable_urls() or self.fleet.urls())
            # prefill / decode disaggregation: these engines only prefill; the client hands their pages to the decoders
            box.append(",".join(self.fleet.urls(worker_type="prefill")))
            box.append(None)
            if getattr(a, "use_miles_router", False) and not box[1]:
                # generation goes through one router process; weight updates still address the engines themselves
                box[2] = (self.fleet.start_router(
                    a.rollout_fleet_base_port + len(self.fleet.engines) + 1,
                    failure_threshold=getattr(a, "miles_router_health_check_failure_threshold", None),
                    timeout=getattr(a, "miles_router_timeout", None), max_connections=getattr(a, "miles_router_max_connections", None)))
        box = box + [None] * (3 - len(box))
        if self.ps.world_size > 1:
            dist.broadcast_object_list(box, src=0)
        self.prefill_urls = [u for u in (box[1] or "").split(",") if u]
        self.router_url = box[2]
        return box[0]

    def _connect_remote_engines(self, urls: list) -> None:
        """Disaggregated mode: the engines run in other processes (`engine/server.py`). Generation goes over HTTP, the
        weight update over a process group of its own that the trainer's first rank and the engines join."""
        from .engine.remote import RemoteEngineClient
        from .weight_sync.broadcast import BroadcastWeightUpdater, HttpEngineHandle

        router = getattr(self, "router_url", None) or getattr(self.args, "rollout_router_url", None)
        prefill = list(getattr(self, "prefill_urls", None) or [u for u in (getattr(self.args, "rollout_prefill_urls", None) or "").split(",") if u])
        self.client = RemoteEngineClient([router] if (router and not prefill) else urls, self.tokenizer, prefill_urls=prefill)
        self.rollout_store = None
        sender = self.ps.rank == 0
        if getattr(self.args, "update_weight_transfer_mode", None) == "disk-delta":
            from .weight_sync.disk_delta import DiskDeltaUpdater

            self.weight_updater = DiskDeltaUpdater(
                self.actor, [HttpEngineHandle(u) for u in urls] if sender else [], self.args.update_weight_disk_dir,
                encoding=getattr(self.args, "update_weight_delta_encoding", "xor"),
                checksum_kind=getattr(self.args, "update_weight_delta_checksum", "xxh3-128"))
        elif sender or self.actor.store.ep_size > 1 or getattr(self.actor, "fsdp", False):
            handles = [HttpEngineHandle(u) for u in urls] if sender else []
            self.weight_updater = BroadcastWeightUpdater(
                self.actor, handles, buffer_bytes=int(getattr(self.args, "update_weight_buffer_size", None) or (512 << 20)),
                is_sender=sender)

    def _start_session_servers(self) -> list:
        """The standalone token-in-token-out session servers (``--use-session-server``): they forward to engines that are
        reached over HTTP, so they need ``--rollout-engine-urls`` / a launched fleet (rollouts on the in-process engine
        use the in-process session of ``rollout.generate_hub.agentic`` instead)."""
        from .rollout.session.server import start_session_servers

        if self.engine is not None:
            raise ValueError("--use-session-server needs engines reached over HTTP (--rollout-engine-urls or "
                             "--launch-rollout-fleet); with the in-process engine use the agentic generate function")
        client = self.client

        def generate(input_ids: list, sampling_params: dict) -> dict:
            out = asyncio.run(client.generate({"input_ids": list(input_ids), "sampling_params": dict(sampling_params),
                                               "return_logprob": True}))
            meta = out.get("meta_info", {})
            return {"output_ids": out["output_ids"], "output_token_logprobs": [lp for lp, _ in meta.get("output_token_logprobs", [])],
                    "finish_reason": meta.get("finish_reason", {}).get("type", "stop"), "weight_version": meta.get("weight_version")}

        return start_session_servers(self.args, self.tokenizer, generate)

    def _replica_bytes(self) -> int:
        cfg = self.actor.cfg
        moe_layers = sum(cfg.layer_is_moe(i) for i in range(cfg.num_layers))
        return moe_layers * cfg.num_experts * 3 * cfg.hidden_size * cfg.moe_ffn_hidden_size * 2

    def _replicate_experts_fits(self, kv_bytes) -> bool:
        """A full copy of the experts for the rollout engine, if asked for (default) and if it fits next to the
        trainer's state, the KV cache and an activation reserve."""
        a = self.args
        from .trainer.actor import replica_wanted

        if not self.actor.on_gpu or not replica_wanted(a, self.ps.ep.size) or self.ps.tp.size > 1:
            return False
        replica = self._replica_bytes()
        free_now, total = torch.cuda.mem_get_info(self.actor.device)
        g = self.actor.store.grad.get("expert")
        lend = g.numel() * g.element_size() if (g is not None and getattr(a, "share_kv_grad_memory", True)) else 0
        need = replica + max((kv_bytes or 0) // 2 - lend, 0) + total // 7  # at least half of the wanted KV pool must remain
        ok = torch.tensor([1.0 if free_now >= need else 0.0], device=self.actor.device)
        if self.ps.world_size > 1:
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)  # all ranks take the same path
        return bool(ok.item() > 0)

    def _build_data_source(self):
        return self._build_data_source_for(self.args)

    def _build_data_source_for(self, a):
        """The prompt stream described by ``a`` (the run's arguments, or a copy with another dataset: multi-LoRA adapters)."""
        path = getattr(a, "data_source_path", None) or "miles_b200.rollout.data_source.RolloutDataSourceWithBuffer"
        path = path.replace("miles.rollout.data_source", "miles_b200.rollout.data_source")
        if not getattr(a, "prompt_data", None) and "Synthetic" not in path and getattr(a, "rollout_global_dataset", True):
            path = "miles_b200.rollout.data_source.SyntheticDataSource"
        local = copy.copy(a)
        local.rollout_seed = a.rollout_seed + 7919 * self.rep  # every data-parallel replica draws its own prompt stream
        if getattr(a, "synthetic_vocab_size", None) is None:
            local.synthetic_vocab_size = self.actor.cfg.vocab_size
        return load_function(path)(local, self.tokenizer)

    def _build_rollout_fn(self):
        a = self.args
        path = getattr(a, "rollout_function_path", None)
        if path is None:
            path = "miles_b200.rollout.fully_async_rollout.FullyAsyncRolloutFn" if getattr(a, "fully_async", False) else \
                "miles_b200.rollout.inference_rollout.InferenceRolloutFn"
        obj = load_function(path)
        local = copy.copy(a)
        ws = self.n_rep
        local.rollout_batch_size = max(1, a.rollout_batch_size // ws)
        local.over_sampling_batch_size = max(local.rollout_batch_size, (a.over_sampling_batch_size or a.rollout_batch_size) // ws)
        self.local_args = local
        if isinstance(obj, type):
            return obj(RolloutFnConstructorInput(local, self.data_source, self.client))
        return lambda inp: obj(local, inp.rollout_id, self.data_source, evaluation=inp.evaluation)

    def _resume(self) -> int:
        a = self.args
        if getattr(a, "start_rollout_id", None) is not None:
            start = a.start_rollout_id
        elif getattr(a, "load", None) and self.actor.loaded_rollout_id is not None and not getattr(a, "finetune", False):
            start = self.actor.loaded_rollout_id + 1  # the checkpoint was written after that rollout
        else:
            start = 0
        if start > 0:
            self.data_source.load(start - 1)
        return start

    # ------------------------------------------------------------------ phases
    def generate(self, rollout_id: int) -> tuple:
        a = self.args
        t0 = time.perf_counter()
        if getattr(a, "load_debug_rollout_data", None):
            blob = torch.load(a.load_debug_rollout_data.format(rollout_id=rollout_id), weights_only=False)
            from .utils.types import Sample

            samples = [Sample.from_dict(d) for d in blob["samples"]]
            ratio = getattr(a, "load_debug_rollout_data_subsample", None)
            if ratio is not None:  # keep the head and the tail of the recording (reference: ray/rollout/debug_data.py:93-99)
                k = int(len(samples) * ratio)
                samples = samples[:k // 2] + samples[len(samples) - (k - k // 2):]
            samples = samples[self.rep::self.n_rep] if self.n_rep > 1 else samples
            return samples, {}
        released = self._release_groups_for_rollout()
        out = self.rollout_fn(RolloutFnTrainInput(rollout_id))
        if asyncio.iscoroutine(out):
            out = asyncio.run(out)
        if self.engine is not None:
            self.engine.drain()  # expert-parallel ranks keep serving dummy iterations until all are done
        if released:
            from .parallel.reloadable_groups import registry

            registry().reload()
        samples = flatten_groups(out.samples if hasattr(out, "samples") else out)
        if getattr(a, "ci_inject_rollout_data_path", None):
            from .utils.ci_checks import inject_rollout_data

            samples = inject_rollout_data(a, rollout_id, samples, self.rep, self.n_rep)
        if getattr(a, "rollout_data_postprocess_path", None):
            # user hook on the generated samples before they become training data (reference signature: fn(args, samples))
            res = load_function(a.rollout_data_postprocess_path)(a, samples)
            samples = res if res is not None else samples
        samples = postprocess_rollout_data(self.local_args, samples)
        # the ranks of a context-parallel group and the stages of a pipeline train on the same samples: each of
        # them generated a share with its own engine, now they pool them
        for axis in (self.ps.cp, self.ps.pp):
            if axis.size > 1:
                samples = self._pool_samples(samples, axis)
        dt = time.perf_counter() - t0
        metrics = dict(getattr(out, "metrics", {}) or {})
        hook = getattr(a, "custom_rollout_log_function_path", None)
        # a user log function may take over (it returns True to suppress the built-in rollout metrics)
        if not (hook and load_function(hook)(rollout_id, a, samples, metrics, dt)):
            metrics.update(compute_rollout_metrics(a, samples, dt))
        if getattr(a, "save_debug_trajectory_data", None):
            self._save_trajectories(rollout_id, samples, evaluation=False)
        if getattr(a, "save_debug_rollout_data", None):
            p = a.save_debug_rollout_data.format(rollout_id=rollout_id)
            os.makedirs(os.path.dirname(p) or ".", exist_ok=True)
            gathered = [[s.to_dict() for s in samples]]
            if self.ps.world_size > 1:
                gathered = [None] * self.ps.world_size
                dist.all_gather_object(gathered, [s.to_dict() for s in samples])
            if self.ps.rank == 0:
                torch.save({"rollout_id": rollout_id, "samples": [d for g in gathered for d in g]}, p)
        return samples, metrics

    def _release_groups_for_rollout(self) -> bool:
        """``--reload-process-groups``: while this rank's engine generates on its own (no lockstep with other ranks) the
        trainer's communicators only pin device memory: destroy them for the rollout and build them again before the
        first collective of the training phase (parallel/reloadable_groups.py)."""
        a = self.args
        if not getattr(a, "reload_process_groups", False) or self.ps.world_size <= 1 or self.engine is None:
            return False
        if getattr(self.engine, "sync", None) is not None or getattr(self.engine, "ep_decode", None) is not None:
            return False  # expert-parallel engines talk to each other while they generate
        from .parallel.reloadable_groups import registry

        freed = registry().release(include_host_groups=self.ps.backend == "gloo")
        self.last_group_release_bytes = freed
        return True

    def _save_trajectories(self, rollout_id: int, samples: list, evaluation: bool) -> None:
        """``--save-debug-trajectory-data TEMPLATE``: one JSON line per sample that carries a conversation
        (``metadata['messages']``), written next to the rollout dump; the messages then leave the sample."""
        import json

        rows = []
        for s in samples:
            msgs = (s.metadata or {}).get("messages")
            if msgs:
                rows.append({"index": s.index, "group_index": s.group_index, "reward": s.reward, "messages": msgs})
        if not rows:
            return
        p = self.args.save_debug_trajectory_data.format(rollout_id=("eval_" if evaluation else "") + str(rollout_id), rank=self.ps.rank)
        os.makedirs(os.path.dirname(p) or ".", exist_ok=True)
        with open(p, "w") as f:
            f.write("".join(json.dumps(r, default=str, separators=(",", ":")) + "\n" for r in rows))
        for s in samples:
            if s.metadata:
                s.metadata.pop("messages", None)

    def _pool_samples(self, samples: list, axis) -> list:
        from .utils.types import Sample

        pooled = [None] * axis.size
        dist.all_gather_object(pooled, [s.to_dict() for s in samples], group=axis.group)
        out, gmap = [], {}
        for part_id, part in enumerate(pooled):
            for d in part:
                smp = Sample.from_dict(d)
                # every rank's data source numbers its groups and samples from zero: make them distinct again
                if smp.group_index is not None:
                    smp.group_index = gmap.setdefault((part_id, smp.group_index), len(gmap))
                if smp.index is not None:
                    smp.index = smp.index * axis.size + part_id
                if smp.rollout_id is not None:
                    smp.rollout_id = smp.rollout_id * axis.size + part_id
                out.append(smp)
        return out

    def offload_rollout(self) -> None:
        if self.engine is not None and self.args.offload_rollout:
            # --offload-rollout-level: "kv_cache" frees the cache (and the graphs that point into it); "weight" is
            # meaningful for engines with weights of their own (a colocated engine reads the trainer's)
            level = getattr(self.args, "offload_rollout_level", None) or ["kv_cache", "weight"]
            tags = tuple(t for t in ("kv_cache",) if t in level) + ("cuda_graph",)
            self.engine.release_memory_occupation(tags)

    def onload_rollout(self) -> None:
        if self.engine is not None and self.args.offload_rollout:
            self.engine.resume_memory_occupation(("kv_cache",))

    def train(self, rollout_id: int, samples: list) -> dict:
        a = self.args
        # the batch travels from the rollout side to the trainer through the object store (in-process by default;
        # --object-store-backend file with --dump-details keeps every batch on disk in the ragged encoding)
        if getattr(self, "object_store", None) is None:
            from .utils.object_store import init_instance

            self.object_store = init_instance(a)
        ref = self.object_store.put(convert_samples_to_train_data(a, samples))
        data = self.object_store.get(ref)
        if not getattr(a, "dump_details", None):
            self.object_store.delete(ref)
        if getattr(a, "balance_data", False) and self.ps.dp.size > 1:
            from .rollout.train_data import rebalance_across_dp

            # the ranks pool their samples and take length-balanced shares (utils/dp_schedule.py)
            data = rebalance_across_dp(self.local_args, data, self.ps.dp.group, self.ps.dp.rank, self.ps.dp.size)
        if self.ft is not None and "train" in self.ft.components:
            return self.ft.train(rollout_id, data)  # through the cell group: retries, suspended cells, scripted faults
        return self._train_once(rollout_id, data)

    def _train_once(self, rollout_id: int, data: dict) -> dict:
        a = self.args
        if getattr(self, "_remerge_before_train", False):
            self.actor.lora.merge()
            self._remerge_before_train = False
        local = copy.copy(self.actor.args)
        metrics = {}
        # every rank already holds exactly its own share: train on it without a DP re-split
        saved = (self.actor.ps.dp_cp.size, self.actor.ps.dp_cp.rank)
        self.actor._local_data = True
        if self.critic is not None:
            metrics.update({k.replace("train/", "train/critic_"): v for k, v in self.critic.train_critic(rollout_id, data).items()})
            if rollout_id < int(getattr(a, "num_critic_only_steps", 0) or 0):
                metrics["train/actor_frozen"] = 1.0  # value-function warm-up: the actor does not train yet
                return metrics
        metrics.update(self.actor.train(rollout_id, data))
        self.h2d_bytes += self.actor.h2d_bytes
        return metrics

    def update_weights(self) -> dict:
        if getattr(self.args, "debug_skip_weight_update", False):
            return {}
        lora = getattr(self.actor, "lora", None)
        if lora is not None and getattr(self.args, "lora_train_only", False):
            # --lora-train-only: the engines keep serving the frozen base policy; the merged adapter is taken out of the
            # live weights for the hand-off and put back for the next training step
            for n, b in lora.base.items():
                self.actor.store.params[n].copy_(b)
            try:
                return self._update_weights()
            finally:
                if self.engine is None or self.engine.store is not self.actor.store:
                    lora.merge()
                else:
                    self._remerge_before_train = True  # shared weights: merge again right before training
        return self._update_weights()

    def _update_weights(self) -> dict:
        if getattr(self.args, "rollout_engine_urls", None):
            out = self.weight_updater.update() if self.weight_updater is not None else {}
            fmt = getattr(self.args, "weight_sync_quant", "none")
            if fmt != "none" and self.ps.rank == 0:
                # --weight-sync-quant: the engines re-quantise what just arrived and serve from the block-scaled copies
                from .weight_sync.broadcast import HttpEngineHandle

                for u in [x for x in self.args.rollout_engine_urls.split(",") if x]:
                    HttpEngineHandle(u).post("/requantize_weights", {"format": fmt})
            if self.ps.world_size > 1:
                dist.barrier()  # nobody generates with the old weights while the first rank is still sending
            return out
        if self.engine is None:
            return {}
        return self.actor.update_weights()

    # ------------------------------------------------------------------ one step / whole run
    def step(self, rollout_id: int) -> dict:
        a = self.args
        T = Timer()
        t0 = time.perf_counter()
        metrics: dict = {}
        hp = getattr(self, "host_profiler", None)
        if hp is not None:
            hp.mark("rollout")
        samples, m = self.generate(rollout_id)
        metrics.update(m)
        t1 = time.perf_counter()
        if getattr(a, "debug_rollout_only", False):
            return metrics
        self.offload_rollout()
        if a.offload_train:
            self.actor.wake_up()
        if hp is not None:
            hp.mark("train")
        metrics.update(self.train(rollout_id, samples))
        if getattr(a, "ci_test", False):
            from .utils.ci_checks import check_rollout_logprobs

            check_rollout_logprobs(a, metrics)
        t2 = time.perf_counter()
        if should_run_periodic_action(rollout_id, a.save_interval, None, a.num_rollout) or self._save_triggered():
            self.actor.save_model(rollout_id)
            self.data_source.save(rollout_id)
        if a.offload_train:
            self.actor.sleep()
        self.onload_rollout()
        if hp is not None:
            hp.mark("update_weights")
        if (rollout_id + 1) % (a.update_weights_interval or 1) == 0:
            metrics.update(self.update_weights())
        t3 = time.perf_counter()
        n_tok = sum(len(s.tokens) for s in samples)
        tot = torch.tensor([float(n_tok)], device=self.actor.device)
        if self.ps.dp.size > 1:
            dist.all_reduce(tot, group=self.ps.dp.group)  # one count per replica (its cp / pp / tp ranks hold the same samples)
        metrics.update({"perf/rollout_time": t1 - t0, "perf/train_time": t2 - t1, "perf/update_weights_wall": t3 - t2,
                        "perf/step_time": t3 - t0, "perf/step_tokens": float(tot.item()),
                        "perf/grpo_tokens_per_s": float(tot.item()) / max(t3 - t0, 1e-9)})
        if a.eval_interval is not None and should_run_periodic_action(rollout_id, a.eval_interval, None, a.num_rollout):
            metrics.update(self.evaluate(rollout_id))
        if self.ft is not None:
            self.ft.after_rollout(rollout_id)
        if self.tracker is not None:
            self.tracker.log(metrics, step=rollout_id)
        return metrics

    def _save_triggered(self) -> bool:
        """``--save-trigger-sentinel PATH``: an operator touches the file to ask for a checkpoint at the next save point;
        the file is removed once seen (every rank takes the first rank's answer)."""
        path = getattr(self.args, "save_trigger_sentinel", None)
        if not path:
            return False
        hit = [False]
        if self.ps.rank == 0 and os.path.exists(path):
            hit[0] = True
            try:
                os.remove(path)
            except OSError:
                pass
        if self.ps.world_size > 1:
            dist.broadcast_object_list(hit, src=0)
        return bool(hit[0])

    # ------------------------------------------------------------------ checkpoint evaluation in the background
    def _checkpoint_eval(self, rollout_id: int, fn_cls) -> dict:
        """``--eval-function-path`` names a :class:`CheckpointEvalFn`: the weights are exported as an HF snapshot under
        ``--eval-hf-dir`` and scored in the background while training goes on (``--eval-max-in-flight``,
        ``--eval-overflow-policy``, ``--eval-keep-snapshots``; ``--eval-num-gpus`` / ``--eval-num-gpus-per-engine`` are
        handed to the evaluator, which owns its engines). Results arrive in the metrics of a later step."""
        import threading

        from .rollout.eval_dispatch import EvalDispatcher

        a = self.args
        if getattr(self, "_eval_rt", None) is None:
            evaluator = fn_cls(a)
            evaluator.num_gpus = int(getattr(a, "eval_num_gpus", 0) or 0)
            evaluator.num_gpus_per_engine = int(getattr(a, "eval_num_gpus_per_engine", 1) or 1)
            ev_loop = asyncio.new_event_loop()
            threading.Thread(target=ev_loop.run_forever, name="eval-dispatch", daemon=True).start()
            box: list = []

            async def export(rid: int, d: str) -> None:
                pass  # the snapshot is written by the training thread before dispatch (it owns the device)

            disp = EvalDispatcher(evaluator, export_fn=export, on_result=lambda rid, m: box.append((rid, m)),
                                  max_in_flight=int(getattr(a, "eval_max_in_flight", 2) or 1),
                                  overflow_policy=getattr(a, "eval_overflow_policy", "backpressure"),
                                  keep_snapshots=int(getattr(a, "eval_keep_snapshots", 2) or 0))
            self._eval_rt = (ev_loop, disp, box, evaluator)
        ev_loop, disp, box, _ = self._eval_rt
        base = getattr(a, "eval_hf_dir", None) or os.path.join(getattr(a, "save", None) or ".", "eval_snapshots")
        d = os.path.join(base, f"rollout_{rollout_id}")
        from .checkpoint import export_hf

        export_hf(self.actor, d)  # every rank takes part; the first rank writes
        if self.ps.rank == 0:
            asyncio.run_coroutine_threadsafe(disp.dispatch(rollout_id, d), ev_loop).result()
        out: dict = {}
        while box:  # whatever has settled since the last call
            rid, m = box.pop(0)
            out.update({(k if k.startswith(("eval/", "perf/")) else f"eval/{k}"): v for k, v in m.items()})
            out["eval/scored_rollout_id"] = rid
        return out

    def drain_evaluations(self) -> dict:
        rt = getattr(self, "_eval_rt", None)
        if rt is None or self.ps.rank != 0:
            return {}
        ev_loop, disp, box, evaluator = rt
        asyncio.run_coroutine_threadsafe(disp.drain(), ev_loop).result()
        evaluator.dispose()
        out: dict = {}
        while box:
            rid, m = box.pop(0)
            out.update({(k if k.startswith(("eval/", "perf/")) else f"eval/{k}"): v for k, v in m.items()})
        return out

    def evaluate(self, rollout_id: int) -> dict:
        fn_path = getattr(self.args, "eval_function_path", None)
        if fn_path:
            from .rollout.eval_dispatch import is_checkpoint_eval_fn

            obj = load_function(fn_path)
            if is_checkpoint_eval_fn(obj):
                metrics = self._checkpoint_eval(rollout_id, obj)
                if self.metric_checker is not None and metrics:
                    self.metric_checker.update(metrics)
                return metrics
        out = self.rollout_fn(RolloutFnEvalInput(rollout_id))
        if asyncio.iscoroutine(out):
            out = asyncio.run(out)
        metrics = dict(getattr(out, "metrics", {}) or {})
        hook = getattr(self.args, "custom_eval_rollout_log_function_path", None)
        if hook:  # reference signature: fn(rollout_id, args, data, extra_metrics) -> bool
            load_function(hook)(rollout_id, self.args, getattr(out, "data", None), metrics)
        if self.metric_checker is not None:
            self.metric_checker.update(metrics)
        return metrics

    def run(self) -> list:
        a = self.args
        history = []
        if (self.engine is not None or getattr(a, "rollout_engine_urls", None)) and not getattr(a, "debug_skip_weight_update", False):
            self.update_weights()  # engines start from the trainer's weights
        if a.eval_interval is not None and not getattr(a, "skip_eval_before_train", False) and self.start_rollout_id == 0:
            self.evaluate(-1)
        profiler = None
        if getattr(a, "use_pytorch_profiler", False) or getattr(a, "memory_snapshot_dir", None):
            from .utils.profile_utils import TrainProfiler

            profiler = TrainProfiler(a, self.ps.rank)  # torch profiler trace of steps [start, end), memory snapshot
        self.host_profiler = None
        if getattr(a, "profile_host_memory", None) and self.ps.rank == 0:
            from .tools.host_memory_profiler import HostMemoryProfiler

            # machine-wide and per-process host memory over time, with a mark per phase (tools/host_memory_profiler.py)
            self.host_profiler = HostMemoryProfiler(a.profile_host_memory, float(getattr(a, "profile_host_memory_interval", 0.5))).start()
        for rid in range(self.start_rollout_id, a.num_rollout):
            if profiler is not None:
                profiler.step(rid - 1)
            m = self.step(rid)
            history.append(m)
            if self.ps.rank == 0:
                keys = ("rollout/raw_reward/mean", "train/pg_loss", "train/grad_norm", "train/train_rollout_logprob_abs_diff",
                        "perf/step_time", "perf/grpo_tokens_per_s")
                print(f"[rollout {rid}] " + " ".join(f"{k.split('/')[-1] if k.count('/')==1 else k}={m[k]:.5g}" for k in keys if k in m), flush=True)
            if getattr(a, "debug_exit_after_rollout", None) is not None and rid >= a.debug_exit_after_rollout:
                break
        if profiler is not None:
            profiler.step(a.num_rollout - 1)  # closes a trace that runs to the last step
        if self.host_profiler is not None:
            self.host_profiler.stop()
        from .checkpoint import wait_for_async_save

        wait_for_async_save()  # a background save must be complete before the job ends
        tail = self.drain_evaluations()
        if tail and history:
            history[-1].update(tail)
            if self.metric_checker is not None:
                self.metric_checker.update(tail)
        if self.ft is not None:
            self.ft.stop()
        if self.metric_checker is not None:
            self.metric_checker.finalize()
        if getattr(a, "enable_event_analyzer", False) and self.actor.events is not None:
            # every replica reported the same weights per step, every sample was trained exactly once
            from .utils.audit import analyze, read_events

            evs = read_events(a.save_debug_event_data) if getattr(a, "save_debug_event_data", None) else self.actor.events.events
            problems = analyze(evs)
            assert not problems, "event analyzer: " + "; ".join(problems[:5])
        return history
