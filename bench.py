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
reads of sampled tokens and metrics (``e2e``).  Rank 0 prints one JSON line.
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
        sm = sorted(float(s[1]) for s in self.samples if s[1].replace(".", "").isdigit())
        mx = [float(s[2]) for s in self.samples if s[2].replace(".", "").isdigit()]
        reasons = set()
        for s in self.samples:
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), s[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(self.samples)}


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
        "--adam-beta2", "0.98", "--clip-grad", "1.0", "--use-dynamic-batch-size", "--max-tokens-per-gpu", str(ns.max_tokens_per_gpu),
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
    t_start = time.perf_counter()
    args = parse_args(flags)
    args.synthetic_prompt_len = ns.prompt_len
    loop = RLLoop(args)
    dev = loop.actor.device
    loop.update_weights()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def launches() -> int:
        n = getattr(loop.actor.model, "launches", 0)
        if loop.actor.opt is not None:
            n += loop.actor.opt.launches
        return n

    def note(msg: str) -> None:  # progress on stderr; stdout carries only the JSON line
        if rank == 0:
            print(f"[bench +{time.perf_counter() - t_start:7.1f}s] {msg}", file=sys.stderr, flush=True)

    note(f"initialised: plan={loop.actor.plan.get('name')} mem={torch.cuda.memory_allocated(dev) / 2**30:.1f} GiB")
    for i in range(ns.warmup):
        m = loop.step(i)
        note(f"warm-up step {i}: rollout {m.get('perf/rollout_time', 0):.1f}s train {m.get('perf/train_time', 0):.1f}s "
             f"peak mem {torch.cuda.max_memory_allocated(dev) / 2**30:.1f} GiB")
    barrier()
    sampler = ClockSampler(int(os.environ.get("LOCAL_RANK", "0")))
    if rank == 0:
        sampler.start()
    l0, h2d0 = launches(), loop.actor.h2d_bytes + (loop.actor.opt.h2d_bytes if loop.actor.opt else 0)
    d2h0 = (loop.engine.d2h_bytes if loop.engine else 0) + (loop.actor.opt.d2h_bytes if loop.actor.opt else 0)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t0 = time.perf_counter()
    ev0.record()
    tokens = 0.0
    last = {}
    for i in range(ns.warmup, ns.warmup + ns.steps):
        last = loop.step(i)
        tokens += last["perf/step_tokens"]
        note(f"timed step {i}: rollout {last.get('perf/rollout_time', 0):.1f}s train {last.get('perf/train_time', 0):.1f}s")
    ev1.record()
    barrier()
    wall = time.perf_counter() - t0
    dev_s = ev0.elapsed_time(ev1) / 1e3
    clocks = sampler.stop() if rank == 0 else {}
    t = torch.tensor([dev_s, wall], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_s, wall = float(t[0]), float(t[1])
    h2d = loop.actor.h2d_bytes + (loop.actor.opt.h2d_bytes if loop.actor.opt else 0) - h2d0
    d2h = (loop.engine.d2h_bytes if loop.engine else 0) + (loop.actor.opt.d2h_bytes if loop.actor.opt else 0) - d2h0
    if rank == 0:
        cfg = loop.actor.cfg
        out = {
            "metric": f"GRPO tokens/s/step (prompt+response tokens / (rollout + logprob + train + weight sync)), {cfg.name}",
            "value": tokens / dev_s, "unit": "tokens/s", "n_gpus": world, "steps": ns.steps, "warmup": ns.warmup,
            "ms_per_step": dev_s * 1e3 / ns.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16" if ns.rollout_quantization == "none" else f"bf16 training, {ns.rollout_quantization} rollout GEMMs", "data": "synthetic (uniform random 1024-token prompts, random-init weights, forced log-normal response lengths)",
            "config": {
                "model": cfg.name, "params_b": round(cfg.num_params() / 1e9, 2), "global_batch": n_prompts * ns.samples_per_prompt,
                "prompts": n_prompts, "samples_per_prompt": ns.samples_per_prompt, "seq_len": ns.prompt_len + ns.max_response_len,
                "prompt_len": ns.prompt_len, "max_response_len": ns.max_response_len, "mean_response_len": ns.mean_response_len,
                "tokens_per_step": tokens / ns.steps, "parallelism": (f"pp{ns.pp} x dp{world // ns.pp}, colocated engine" if ns.pp > 1 else
                                                     f"dp{world}-attn x ep{world}-experts, colocated engine" if ns.tp == 1 else
                                                     f"tp{ns.tp} x dp{world // ns.tp}, colocated engine"),
                "optimizer_plan": loop.actor.plan.get("name"), "routing_replay": not ns.no_routing_replay,
                "l2": f"working set ({cfg.num_params() * 2 / 1e9:.0f} GB of weights + KV cache) is far larger than L2; no explicit flush",
                "phases_s": {k: round(float(v), 3) for k, v in last.items() if k.startswith("perf/") and k.endswith(("_time", "_wall"))},
            },
            "clocks": clocks,
            "e2e": {"value": tokens / wall, "unit": "tokens/s", "h2d_bytes_per_step": h2d / ns.steps,
                    "d2h_bytes_per_step": d2h / ns.steps},
            "gpu_launches": launches() - l0,
            "train_rollout_logprob_abs_diff": last.get("train/train_rollout_logprob_abs_diff"),
        }
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
