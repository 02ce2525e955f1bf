"""Expert-parallel MoE layer benchmark: NCCL all-to-all baseline vs NVLink peer-memory exchange vs the same with
the return transfer fused into the grouped-GEMM epilogue.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29555 \
        benchmarks/bench_ep.py --tokens 8192

Times one MoE block (router, dispatch, grouped GEMMs, return, combine) forward and forward+backward with CUDA
events, max over ranks, after warm-up; inputs are far larger than L2. The roofline printed for the fused path is
max(FLOPs / measured bf16 peak, bytes over NVLink / 770 GB/s per direction).
"""
from __future__ import annotations

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import argparse
import json
import os

import torch
import torch.distributed as dist


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192, help="tokens per rank")
    ap.add_argument("--model", default="qwen3-30B-A3B")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--bf16-tflops", type=float, default=1339.5, help="measured sustained cuBLAS bf16 TFLOP/s")
    ns = ap.parse_args()

    from miles_b200.models import ParamStore, build_model, get_config
    from miles_b200.parallel.expert_parallel import ExpertParallel
    from miles_b200.parallel.state import init_parallel_state

    world = int(os.environ.get("WORLD_SIZE", "1"))
    ps = init_parallel_state(ep=world)
    dev = ps.device
    cfg = get_config(ns.model)
    cfg.num_layers = 1
    store = ParamStore(cfg, dev, torch.bfloat16, ep_size=world, ep_rank=ps.ep.rank, init_std=0.02, seed=1)
    store.allocate_grads(torch.float32, torch.bfloat16)
    T, H, K = ns.tokens, cfg.hidden_size, cfg.moe_top_k
    g = torch.Generator().manual_seed(7 + ps.rank)
    h2 = (torch.randn(T, H, generator=g) * 0.5).to(dev).to(torch.bfloat16)
    dy = (torch.randn(T, H, generator=g) * 0.01).to(dev).to(torch.bfloat16)
    results = {}
    for mode in ("nccl", "fused_copy", "fused"):
        ep = ExpertParallel(cfg, ps, fused=mode != "nccl", max_tokens=T, fused_epilogue=mode == "fused")
        model = build_model(cfg, store, "b200", ep=ep)

        def fwd():
            return model.moe_forward(0, h2, None, None, keep=False)

        def fwd_bwd():
            _, saved = model.moe_forward(0, h2, None, None, keep=True)
            return model.moe_backward(0, h2, dy, saved)

        for name, fn in (("fwd", fwd), ("fwd_bwd", fwd_bwd)):
            for _ in range(3):
                fn()
            dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(ns.iters):
                fn()
            e1.record()
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1) / ns.iters], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            results[f"{mode}/{name}_ms"] = round(float(t), 4)
        model.check_status()
        ep.check_status()
        del model, ep
        torch.cuda.empty_cache()
    if ps.rank == 0:
        I = cfg.moe_ffn_hidden_size
        flops_fwd = 2.0 * T * K * H * 3 * I  # per rank on average (balanced routing)
        remote = (world - 1) / world
        nvlink_bytes = T * K * H * 2 * remote  # per direction, per transfer
        t_gemm = flops_fwd / (ns.bf16_tflops * 1e12) * 1e3
        t_link = 2 * nvlink_bytes / 770e9 * 1e3  # dispatch + return
        results["roofline_fwd_ms"] = round(max(t_gemm, t_link), 4)
        results["roofline_parts_ms"] = {"gemm": round(t_gemm, 4), "nvlink": round(t_link, 4)}
        results["config"] = {"model": ns.model, "tokens_per_rank": T, "world": world, "top_k": K}
        print(json.dumps(results))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
