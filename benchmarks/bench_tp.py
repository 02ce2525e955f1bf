"""Row-parallel projection + all-reduce: one fused kernel (GEMM epilogue pushes partial sums to the peers) vs
local GEMM followed by NCCL all-reduce.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29556 \
        benchmarks/bench_tp.py --tokens 8192

Shapes default to Qwen3-4B under TP = world size (o projection and MLP down projection). CUDA events, max over
ranks, after warm-up; operands exceed L2. Roofline = max(FLOPs / measured bf16 peak, bytes over NVLink / 770 GB/s).
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
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=2560)
    ap.add_argument("--attn-dim", type=int, default=4096)
    ap.add_argument("--ffn", type=int, default=9728)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--bf16-tflops", type=float, default=1339.5)
    ns = ap.parse_args()
    from miles_b200.parallel.state import init_parallel_state
    from miles_b200.parallel.tensor_parallel import TensorParallel

    world = int(os.environ.get("WORLD_SIZE", "1"))
    ps = init_parallel_state()
    dev = ps.device
    T, H = ns.tokens, ns.hidden
    out = {}
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    for name, k_full in (("o_proj", ns.attn_dim), ("mlp_down", ns.ffn)):
        kl = k_full // world
        a = (torch.randn(T, kl, device=dev) * 0.5).to(torch.bfloat16)
        w = (torch.randn(H, kl, device=dev) * 0.05).to(torch.bfloat16)
        res = torch.randn(T, H, device=dev).to(torch.bfloat16)
        for mode in ("nccl", "fused"):
            tp = TensorParallel(dist.group.WORLD, ps.rank, world, dev, H, T, fused=mode == "fused")
            for _ in range(3):
                tp.linear_allreduce(a, w, residual=res, gemm_status=status)
            dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(ns.iters):
                tp.linear_allreduce(a, w, residual=res, gemm_status=status)
            e1.record()
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1) / ns.iters], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            out[f"{name}/{mode}_ms"] = round(float(t), 4)
            tp.check_status()
            del tp
        t_gemm = 2.0 * T * kl * H / (ns.bf16_tflops * 1e12) * 1e3
        t_link = (world - 1) * T * H * 2 / 770e9 * 1e3
        out[f"{name}/roofline_ms"] = round(max(t_gemm, t_link), 4)
        out[f"{name}/roofline_parts_ms"] = {"gemm": round(t_gemm, 4), "nvlink": round(t_link, 4)}
    if ps.rank == 0:
        out["config"] = {"tokens": T, "hidden": H, "world": world}
        print(json.dumps(out))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
