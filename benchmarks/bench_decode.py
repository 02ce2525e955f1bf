"""Decode-step latency of the rollout engine by batch size, against the bytes a step has to stream.

    python benchmarks/bench_decode.py --model qwen3-30B-A3B --layers 8 --batches 1,2,4,8,16,32,64 --ctx 2000

Builds the model with the real layer shapes but ``--layers`` decoder layers (a decode step is the same kernel
sequence per layer, so microseconds per layer carry over to the full depth), fills the KV cache with ``--ctx``
positions per sequence, and replays the engine's own captured decode graph. Per batch size one JSON line: ms per
step, microseconds per layer, the bytes one layer streams from HBM at that batch (attention projections, router,
the experts the batch touches in expectation, KV rows) and the fraction of the measured copy bandwidth
(``--hbm-gbs``, default from MEASURED_PEAKS.json) that corresponds to. SM clocks are sampled during the timed loops.
"""
from __future__ import annotations

import argparse
import copy
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen3-30B-A3B")
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--batches", default="1,2,4,8,16,32,64")
    ap.add_argument("--ctx", type=int, default=2000)
    ap.add_argument("--steps", type=int, default=60)
    ap.add_argument("--hbm-gbs", type=float, default=None)
    ns = ap.parse_args()

    from clocks import ClockSampler
    from miles_b200.engine import Engine, SamplingParams
    from miles_b200.models import ParamStore, build_model, get_config

    hbm = ns.hbm_gbs
    if hbm is None:
        try:
            hbm = json.load(open(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")))["hbm_gbs"]
        except Exception:  # noqa: BLE001
            hbm = 6650.0  # fallback figure of this pool
    dev = torch.device("cuda")
    cfg = copy.copy(get_config(ns.model))
    cfg.num_layers = ns.layers
    store = ParamStore(cfg, dev, torch.bfloat16)
    model = build_model(cfg, store, "b200")
    batches = [int(b) for b in ns.batches.split(",")]
    eng = Engine(model, max_running=max(batches), page_size=64, max_seq_len=ns.ctx + ns.steps * 4 + 64, use_cuda_graph=True)
    g = torch.Generator().manual_seed(0)
    H, D = cfg.hidden_size, cfg.head_dim
    attn_w = (cfg.qkv_dim * H + H * cfg.q_dim) * 2
    expert_w = 3 * H * cfg.moe_ffn_hidden_size * 2 if cfg.is_moe else 0
    for B in batches:
        prompts = [torch.randint(0, cfg.vocab_size, (ns.ctx,), generator=g).tolist() for _ in range(B)]
        for p in prompts:
            eng.add_request(p, SamplingParams(temperature=1.0, max_new_tokens=ns.steps * 3 + 8, ignore_eos=True, sampling_seed=1))
        while eng.waiting:
            eng.step()          # prefill
        for _ in range(5):
            eng.step()          # graph capture + warm-up
        torch.cuda.synchronize()
        sampler = ClockSampler(torch.cuda.current_device())
        sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(ns.steps):
            eng.step()
        eng._drain_pending()
        e1.record()
        torch.cuda.synchronize()
        clocks = sampler.stop()
        ms = e0.elapsed_time(e1) / ns.steps
        eng.abort_request(abort_all=True)
        eng.pop_finished()
        if cfg.is_moe:
            touched = cfg.num_experts * (1.0 - (1.0 - cfg.moe_top_k / cfg.num_experts) ** B)
            layer_bytes = attn_w + cfg.num_experts * H * 2 + touched * expert_w
        else:
            layer_bytes = attn_w + 3 * H * cfg.ffn_hidden_size * 2
        layer_bytes += B * ns.ctx * 2 * cfg.num_kv_heads * D * 2
        head_bytes = cfg.vocab_size * H * 2
        floor_ms = (ns.layers * layer_bytes + head_bytes) / (hbm * 1e9) * 1e3
        print(json.dumps({"what": "decode_step", "model": ns.model, "layers": ns.layers, "batch": B, "ctx": ns.ctx, "ms_per_step": ms,
                          "us_per_layer": (ms - head_bytes / (hbm * 1e9) * 1e3) * 1e3 / ns.layers, "layer_mbytes": layer_bytes / 1e6,
                          "hbm_floor_ms": floor_ms, "frac_of_measured_hbm": floor_ms / ms,
                          "clocks": clocks}), flush=True)


if __name__ == "__main__":
    main()
