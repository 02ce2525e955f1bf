"""Headline benchmark: GRPO tokens/s of one full RL step (rollout + log-prob recompute + train + weight
sync) on Qwen3-30B-A3B, random-init weights, synthetic prompts.

    python bench.py --gpus 1 --steps 2 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus 8 --steps 2 --warmup 3

Weak scaling: every GPU handles 8 prompts x 8 samples (64 prompts x 8 samples at 8 GPUs, the batch of
the 30B-A3B GRPO recipe), 1024-token prompts, responses of up to 8192 tokens whose lengths follow a
seeded log-normal (random-init weights never emit EOS, so lengths are forced like the reference's
benchmark generate function does).  The step is driven through the public ``RLLoop.step`` API.  Two
clocks are taken around the same K steps: CUDA events on the main stream (``value``) and the host wall
clock around the API call including prompt creation, pinned-host staging, H2D copies and the D2H
reads of sampled tokens and metrics (``e2e``).  Rank 0 prints one cumulative JSON line after every timed
step (the last line is the result, so a run that is cut short still leaves a parsed value).  The run keeps
inside a wall-clock budget (``--budget-s``, 760 s from process start by default): when the requested warm-up
and step counts do not fit, warm-up is cut first (to three, at least one), then the timed steps (at least two);
the configuration is never shrunk and ``steps`` / ``warmup`` report what really ran.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def reference_arm(ns) -> None:
    """The reference cannot run on this image: its trainer and engine are Megatron-LM, TransformerEngine,
    SGLang and Ray, none of which is installed or installable offline."""
    why = ("reference installed with --no-deps under baseline/_ref but cannot run: its train.py imports ray, "
           "megatron.core, transformer_engine and sglang, which are absent from the image and the offline wheelhouse")
    try:
        sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline", "_ref"))
        import importlib

        importlib.import_module("miles.ray.placement_group")
        why = "reference imported unexpectedly but needs a Ray cluster and SGLang servers that do not exist here"
    except Exception as e:  # noqa: BLE001
        why += f" ({type(e).__name__}: {str(e)[:80]})"
    print(json.dumps({"impl": "reference", "unavailable": why}))


class ClockSampler(threading.Thread):
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        super().__init__(daemon=True)
        self.gpu = gpu_index
        self.samples = []
        self._stop_evt = threading.Event()
        self.proc = None

    def run(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                                          "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            for line in self.proc.stdout:
                if self._stop_evt.is_set():
                    break
                parts = [p.strip() for p in line.split(",")]
                if len(parts) >= 9:
                    self.samples.append(parts)
        except Exception:
            pass

    def stop(self) -> dict:
        self._stop_evt.set()
        if self.proc is not None:
            self.proc.terminate()
        return self.snapshot()

    def snapshot(self) -> dict:
        sm = sorted(float(s[1]) for s in self.samples if s[1].replace(".", "").isdigit())
        mx = [float(s[2]) for s in self.samples if s[2].replace(".", "").isdigit()]
        reasons = set()
        for s in list(self.samples):
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), s[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(self.samples)}


def plan_warmup(done: int, est_s: float, left_s: float, want_warmup: int, want_steps: int, min_timed: int = 2) -> int:
    """How many warm-up steps to run in total, decided after ``done`` of them, when a step takes ``est_s`` and
    ``left_s`` seconds of the wall-clock budget remain. Everything requested if it fits; otherwise warm-up is cut
    first (not below three while three warm-up plus ``min_timed`` timed steps fit, never below one) and the timed
    steps afterwards."""
    feasible = done + int(left_s // max(est_s, 1e-6))
    if feasible >= want_warmup + want_steps:
        return want_warmup
    target = min(max(feasible - want_steps, min(3, want_warmup)), want_warmup)
    if feasible - target < min_timed:
        target = max(1, feasible - min_timed)
    return max(target, 1)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--model", default="qwen3-30B-A3B")
    ap.add_argument("--prompts-per-gpu", type=int, default=8)
    ap.add_argument("--samples-per-prompt", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=1024)
    ap.add_argument("--max-response-len", type=int, default=8192)
    ap.add_argument("--mean-response-len", type=float, default=2048.0)
    ap.add_argument("--max-tokens-per-gpu", type=int, default=32768)
    ap.add_argument("--no-routing-replay", action="store_true")
    ap.add_argument("--tp", type=int, default=1, help="tensor-parallel size (dense models; the rest of the GPUs are data parallel)")
    ap.add_argument("--rollout-quantization", default="none", choices=["none", "mxfp8", "nvfp4"],
                    help="serve the rollout from block-scaled copies of the weights (not the headline configuration)")
    ap.add_argument("--pp", type=int, default=1, help="pipeline-parallel size (experts are then not expert parallel)")
    ap.add_argument("--budget-s", type=float, default=float(os.environ.get("BENCH_BUDGET_S", 760)),
                    help="wall-clock seconds from process start within which the run must end: warm-up and timed steps "
                         "are cut (never the configuration) when the requested counts would not fit; the steps really "
                         "timed are reported in `steps`")
    ap.add_argument("--replicate-experts", choices=["auto", "on", "off"], default="auto",
                    help="rollout engine of an expert-parallel run: full replica of the experts per GPU, or expert parallel")
    ns = ap.parse_args()
    if ns.impl == "reference":
        reference_arm(ns)
        return

    import torch
    import torch.distributed as dist

    from miles_b200.loop import RLLoop
    from miles_b200.utils.arguments import parse_args

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    assert world == ns.gpus, f"--gpus {ns.gpus} but WORLD_SIZE={world}; launch with torchrun --nproc-per-node {ns.gpus}"
    n_prompts = ns.prompts_per_gpu * (world // ns.tp)
    flags = [
        "--model-preset", ns.model, "--num-rollout", str(ns.steps + ns.warmup),
        "--rollout-batch-size", str(n_prompts), "--n-samples-per-prompt", str(ns.samples_per_prompt),
        "--rollout-max-prompt-len", str(ns.prompt_len), "--rollout-max-response-len", str(ns.max_response_len),
        "--rollout-temperature", "1.0", "--rm-type", "parity", "--advantage-estimator", "grpo",
        "--eps-clip", "0.2", "--eps-clip-high", "0.28", "--lr", "1e-6", "--weight-decay", "0.1", "--adam-beta1", "0.9",
        "--adam-beta2", "0.98", "--clip-grad", "1.0",
        # fp32 master weights with 16-bit moments (the reference's precision-aware optimizer): the one optimizer
        # format that fits this model at every GPU count of the run, down to a single 192 GB device
        "--use-precision-aware-optimizer", "--exp-avg-dtype", "bf16", "--exp-avg-sq-dtype", "bf16", "--use-dynamic-batch-size", "--max-tokens-per-gpu", str(ns.max_tokens_per_gpu),
        "--actor-num-nodes", "1", "--actor-num-gpus-per-node", str(world), "--colocate",
        "--expert-model-parallel-size", str(world if (ns.tp == 1 and ns.pp == 1) else 1), "--tensor-model-parallel-size", str(ns.tp),
        "--pipeline-model-parallel-size", str(ns.pp),
        "--recompute-granularity", "full",
        "--custom-generate-function-path", "miles_b200.rollout.generate_hub.benchmarkers.generate",
        "--benchmark-mean-response-len", str(ns.mean_response_len), "--sglang-mem-fraction-static", "0.8",
    ]
    if not ns.no_routing_replay:
        flags += ["--use-rollout-routing-replay"]
    if ns.rollout_quantization != "none":
        flags += ["--rollout-quantization", ns.rollout_quantization]
    if ns.replicate_experts != "auto":
        flags += ["--rollout-replicate-experts" if ns.replicate_experts == "on" else "--no-rollout-replicate-experts"]
    args = parse_args(flags)
    args.synthetic_prompt_len = ns.prompt_len

    def note(msg: str) -> None:  # progress on stderr; stdout carries only JSON lines
        if rank == 0:
            print(f"[bench +{time.perf_counter() - T_START:7.1f}s] {msg}", file=sys.stderr, flush=True)

    loop = RLLoop(args)
    dev = loop.actor.device
    loop.update_weights()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def agree(x: float) -> float:
        """The first rank's view of a host-side number, so that every rank takes the same branch."""
        if world == 1:
            return x
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.broadcast(t, src=0)
        return float(t.item())

    models = {id(m): m for m in (loop.actor.model, getattr(loop.engine, "model", None)) if m is not None}

    def launches() -> int:
        n = sum(getattr(m, "launches", 0) for m in models.values())
        if loop.actor.opt is not None:
            n += loop.actor.opt.launches
        return n

    def copied() -> tuple:
        opt = loop.actor.opt
        eng = loop.engine
        h2d = loop.actor.h2d_bytes + (opt.h2d_bytes if opt else 0) + (eng.h2d_bytes if eng else 0)
        d2h = (eng.d2h_bytes if eng else 0) + (opt.d2h_bytes if opt else 0)
        return h2d, d2h

    note(f"initialised: plan={loop.actor.plan.get('name')} mem={torch.cuda.memory_allocated(dev) / 2**30:.1f} GiB")
    budget = ns.budget_s
    left = lambda: budget - (time.perf_counter() - T_START) - 20.0  # 20 s to print, tear down and exit
    warm_target, done, est = ns.warmup, 0, 0.0
    while done < warm_target:
        t_a = time.perf_counter()
        m = loop.step(done)
        barrier()
        est = agree(time.perf_counter() - t_a)
        done += 1
        note(f"warm-up step {done - 1}: {est:.1f}s (rollout {m.get('perf/rollout_time', 0):.1f}s train {m.get('perf/train_time', 0):.1f}s) "
             f"peak mem {torch.cuda.max_memory_allocated(dev) / 2**30:.1f} GiB")
        warm_target = int(agree(plan_warmup(done, est, left(), ns.warmup, ns.steps)))
    warm_run = done
    barrier()
    sampler = ClockSampler(int(os.environ.get("LOCAL_RANK", "0")))
    if rank == 0:
        sampler.start()
    l0 = launches()
    h2d0, d2h0 = copied()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    cfg = loop.actor.cfg
    dtype = ("bf16 compute; fp32 master weights (bf16 weight + 16-bit remainder), bf16 Adam moments (precision-aware "
             "optimizer), fp32 dense / bf16 expert gradient accumulation")
    if loop.actor.plan.get("state") != "bf16" or not loop.actor.plan.get("master"):
        dtype = f"bf16 compute; optimizer plan {loop.actor.plan.get('name')}"
    if ns.rollout_quantization != "none":
        dtype += f"; {ns.rollout_quantization} rollout GEMMs"
    engine_kind = ("expert-parallel engine" if getattr(loop.engine, "ep_decode", None) is not None or getattr(loop.engine, "ep_ll", None) is not None
                   else "full expert replica per GPU" if getattr(loop, "rollout_store", None) is not None else "engine on the trainer's weights")
    barrier()
    t0 = time.perf_counter()
    ev0.record()
    tokens, timed, last = 0.0, 0, {}
    while timed < ns.steps:
        last = loop.step(warm_run + timed)
        ev1.record()
        barrier()  # ends with a device synchronize: ev1 is complete
        wall = time.perf_counter() - t0
        timed += 1
        tokens += last["perf/step_tokens"]
        t = torch.tensor([ev0.elapsed_time(ev1) / 1e3, wall], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dev_s, wall = float(t[0]), float(t[1])
        est = max(est * 0.5, dev_s / timed)
        note(f"timed step {timed - 1}: rollout {last.get('perf/rollout_time', 0):.1f}s train {last.get('perf/train_time', 0):.1f}s")
        if loop.engine is not None and loop.engine.bucket_time:
            note("decode ms/step by row bucket: " + ", ".join(f"{b}: {1e3 * t / max(n, 1):.2f} x{n}"
                                                               for b, (t, n) in sorted(loop.engine.bucket_time.items())))
            loop.engine.bucket_time = {}
        stop = timed >= ns.steps or (timed >= 2 and agree(float(left() < est * 1.1)) > 0)
        h2d, d2h = copied()
        if rank == 0:
            clocks = sampler.stop() if stop else sampler.snapshot()
            out = {
                "metric": f"GRPO tokens/s/step (prompt+response tokens / (rollout + logprob + train + weight sync)), {cfg.name}",
                "value": tokens / dev_s, "unit": "tokens/s", "n_gpus": world, "steps": timed, "warmup": warm_run,
                "steps_requested": ns.steps, "warmup_requested": ns.warmup, "final": bool(stop),
                "ms_per_step": dev_s * 1e3 / timed, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": dtype,
                "data": "synthetic (uniform random 1024-token prompts, random-init weights, forced log-normal response lengths)",
                "config": {
                    "model": cfg.name, "params_b": round(cfg.num_params() / 1e9, 2), "global_batch": n_prompts * ns.samples_per_prompt,
                    "prompts": n_prompts, "samples_per_prompt": ns.samples_per_prompt, "seq_len": ns.prompt_len + ns.max_response_len,
                    "prompt_len": ns.prompt_len, "max_response_len": ns.max_response_len, "mean_response_len": ns.mean_response_len,
                    "tokens_per_step": tokens / timed,
                    "parallelism": (f"pp{ns.pp} x dp{world // ns.pp}, colocated engine" if ns.pp > 1 else
                                    f"dp{world}-attn x ep{world}-experts, colocated {engine_kind}" if ns.tp == 1 else
                                    f"tp{ns.tp} x dp{world // ns.tp}, colocated engine"),
                    "optimizer_plan": loop.actor.plan.get("name"), "routing_replay": not ns.no_routing_replay,
                    "l2": f"working set ({cfg.num_params() * 2 / 1e9:.0f} GB of weights + KV cache) is far larger than L2; no explicit flush",
                    "budget_s": budget, "wall_s_since_start": round(time.perf_counter() - T_START, 1),
                    "phases_s": {k: round(float(v), 3) for k, v in last.items() if k.startswith("perf/") and k.endswith(("_time", "_wall"))},
                },
                "clocks": clocks,
                "e2e": {"value": tokens / wall, "unit": "tokens/s", "h2d_bytes_per_step": h2d / timed - h2d0 / timed,
                        "d2h_bytes_per_step": d2h / timed - d2h0 / timed,
                        "how": "host wall clock around RLLoop.step(): each step creates its prompts on the host, copies them and the "
                               "packed training batches from pinned host memory to the device, and reads the sampled tokens, "
                               "log-probs, routed experts and the step's loss / metrics back to the host, all inside the timed region"},
                "gpu_launches": launches() - l0,
                "train_rollout_logprob_abs_diff": last.get("train/train_rollout_logprob_abs_diff"),
            }
            print(json.dumps(out), flush=True)  # one cumulative line per timed step: the last line is the result
        if stop:
            break
    if world > 1:
        dist.destroy_process_group()


T_START = time.perf_counter()

if __name__ == "__main__":
    main()
