"""Micro-benchmarks of single kernels (CUDA events, warm-up, L2-exceeding operands), also the small cases that
profiler captures are taken on.

    python benchmarks/bench_kernels.py gemm --m 8192 --n 8192 --k 8192
    python benchmarks/bench_kernels.py gemm_mx --kind mxfp8 --m 8192 --n 8192 --k 8192
    python benchmarks/bench_kernels.py attn --seqs 4 --len 8192
    python benchmarks/bench_kernels.py gemv --t 4 --n 49152 --k 2048
    python benchmarks/bench_kernels.py decode_attn --batch 64 --ctx 1500

    python benchmarks/bench_kernels.py attn_bwd --seqs 4 --len 8192 --library

Each prints one JSON line with the time per launch, the achieved TFLOP/s or TB/s, the SM clocks sampled while the
timed loop ran (``clocks``) and ``ms_x_mhz`` (time x median SM MHz, comparable across runs at different clocks).
"""
from __future__ import annotations

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import argparse
import json

import torch


CLOCKS: dict = {}


def _time(fn, iters: int, warmup: int = 3, min_seconds: float = 0.6) -> float:
    """Milliseconds per call (CUDA events around the loop, after warm-up). The loop is repeated until it has run for
    ``min_seconds`` so that the clock sampler sees the kernel under load; the last repetition is the one reported."""
    import time

    from clocks import ClockSampler

    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    sampler = ClockSampler(torch.cuda.current_device())
    sampler.start()
    t0 = time.perf_counter()
    ms = 0.0
    while True:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / iters
        if time.perf_counter() - t0 >= min_seconds or iters <= 2:
            break
    CLOCKS.update(sampler.stop())
    return ms


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemm", "gemm_mx", "attn", "attn_bwd", "gemv", "decode_attn"])
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--t", type=int, default=4)
    ap.add_argument("--seqs", type=int, default=4)
    ap.add_argument("--len", type=int, default=8192)
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--ctx", type=int, default=1500)
    ap.add_argument("--hq", type=int, default=32)
    ap.add_argument("--hk", type=int, default=4)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--block-n", type=int, default=0)
    ap.add_argument("--kind", default="mxfp8", choices=["mxfp8", "nvfp4"])
    ap.add_argument("--library", action="store_true", help="also time the library kernel for the same problem")
    ns = ap.parse_args()
    from miles_b200.ops import _ext

    C = _ext.load(required=True)
    dev = "cuda"
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    out = {"what": ns.what}
    if ns.what == "gemm":
        a = torch.randn(ns.m, ns.k, device=dev, dtype=torch.bfloat16)
        b = torch.randn(ns.n, ns.k, device=dev, dtype=torch.bfloat16)
        c = torch.empty(ns.m, ns.n, device=dev, dtype=torch.bfloat16)
        ms = _time(lambda: C.gemm(a, b, c, False, False, False, 0, status), ns.iters)
        fl = 2.0 * ns.m * ns.n * ns.k
        out.update(shape=[ns.m, ns.n, ns.k], ms=ms, tflops=fl / ms / 1e9)
        if ns.library:
            ml = _time(lambda: torch.matmul(a, b.t(), out=c), ns.iters)
            out.update(library_ms=ml, library_tflops=fl / ml / 1e9)
    elif ns.what == "gemm_mx":
        from miles_b200.ops.mx_gemm import KINDS, quantize_operand

        a = quantize_operand(torch.randn(ns.m, ns.k, device=dev, dtype=torch.bfloat16), ns.kind)
        b = quantize_operand(torch.randn(ns.n, ns.k, device=dev, dtype=torch.bfloat16), ns.kind)
        ms = _time(lambda: C.gemm_mx(a.q, a.atoms, b.q, b.atoms, KINDS[ns.kind], 1.0, 0, None, None, status, ns.block_n), ns.iters)
        fl = 2.0 * ns.m * ns.n * ns.k
        out.update(kind=ns.kind, shape=[ns.m, ns.n, ns.k], ms=ms, tflops=fl / ms / 1e9, status=int(status))
    elif ns.what == "attn":
        from miles_b200.ops.attention import build_tiles

        lens = [ns.len] * ns.seqs
        T = sum(lens)
        qkv = torch.randn(T, ns.hq + 2 * ns.hk, 128, device=dev, dtype=torch.bfloat16)
        q, k, v = qkv[:, :ns.hq], qkv[:, ns.hq:ns.hq + ns.hk], qkv[:, ns.hq + ns.hk:]
        tiles = build_tiles(lens).to(dev)
        ms = _time(lambda: C.flash_attn_fwd(q, k, v, tiles, 128 ** -0.5, status), ns.iters)
        fl = sum(4.0 * 128 * ns.hq * (n * (n + 1) / 2) for n in lens)
        out.update(lens=lens, ms=ms, tflops=fl / ms / 1e9)
        if ns.library:
            from flash_attn import flash_attn_varlen_func

            cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=dev)
            ml = _time(lambda: flash_attn_varlen_func(q, k, v, cu, cu, ns.len, ns.len, softmax_scale=128 ** -0.5, causal=True), ns.iters)
            out.update(library_ms=ml, library_tflops=fl / ml / 1e9)
    elif ns.what == "attn_bwd":
        from miles_b200.ops.attention import build_bwd_blocks, build_tiles

        lens = [ns.len] * ns.seqs
        T = sum(lens)
        qkv = torch.randn(T, ns.hq + 2 * ns.hk, 128, device=dev, dtype=torch.bfloat16)
        q, k, v = qkv[:, :ns.hq].contiguous(), qkv[:, ns.hq:ns.hq + ns.hk], qkv[:, ns.hq + ns.hk:]
        d_o = torch.randn(T, ns.hq, 128, device=dev, dtype=torch.bfloat16)
        o, lse = C.flash_attn_fwd(q, k, v, build_tiles(lens).to(dev), 128 ** -0.5, status)
        blocks = build_bwd_blocks(lens).to(dev)
        ms = _time(lambda: C.flash_attn_bwd(q, k, v, o, d_o, lse, blocks, 128 ** -0.5, status), ns.iters)
        fl = sum(10.0 * 128 * ns.hq * (n * (n + 1) / 2) for n in lens)  # five 2*M*N*K products per (query, key) pair
        out.update(lens=lens, ms=ms, tflops=fl / ms / 1e9)
        if ns.library:
            from flash_attn.flash_attn_interface import _flash_attn_varlen_backward

            cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=dev)
            kc, vc = k.contiguous(), v.contiguous()
            dq, dk, dv = torch.empty_like(q), torch.empty_like(kc), torch.empty_like(vc)
            ml = _time(lambda: _flash_attn_varlen_backward(d_o, q, kc, vc, o, lse, dq, dk, dv, cu, cu, ns.len, ns.len, 0.0,
                                                           128 ** -0.5, True, -1, -1, 0.0, None, False, None, False), ns.iters)
            out.update(library_ms=ml, library_tflops=fl / ml / 1e9)
    elif ns.what == "gemv":
        x = torch.randn(ns.t, ns.k, device=dev, dtype=torch.bfloat16)
        w = torch.randn(ns.n, ns.k, device=dev, dtype=torch.bfloat16)
        y = torch.empty(ns.t, ns.n, device=dev, dtype=torch.bfloat16)
        ms = _time(lambda: C.small_gemv(x, None, 1e-6, w, None, y, status), ns.iters)
        out.update(shape=[ns.t, ns.n, ns.k], ms=ms, tbps=ns.n * ns.k * 2 / ms / 1e9)
    else:
        page, B, ctx = 64, ns.batch, ns.ctx
        pages_per = (ctx + page - 1) // page
        slots = B * pages_per * page + page
        kc = torch.randn(slots, ns.hk, 128, device=dev, dtype=torch.bfloat16)
        vc = torch.randn(slots, ns.hk, 128, device=dev, dtype=torch.bfloat16)
        q = torch.randn(B, ns.hq, 128, device=dev, dtype=torch.bfloat16)
        o = torch.empty_like(q)
        bt = (1 + torch.arange(B * pages_per, dtype=torch.int32, device=dev)).view(B, pages_per)
        sl = torch.full((B,), ctx, dtype=torch.int32, device=dev)
        splits = max(1, min(16, (148 * 3) // max(B * ns.hk, 1)))
        scratch = torch.empty(B * ns.hq * splits * 130, dtype=torch.float32, device=dev)
        ms = _time(lambda: C.paged_decode_attention(q, kc, vc, bt, sl, o, scratch, page, splits, 128 ** -0.5), ns.iters)
        out.update(batch=B, ctx=ctx, splits=splits, ms=ms, tbps=2.0 * B * ctx * ns.hk * 128 * 2 / ms / 1e9)
    out["status"] = int(status.item())
    out["clocks"] = dict(CLOCKS)
    if CLOCKS.get("sm_mhz") and "ms" in out:
        out["ms_x_mhz"] = out["ms"] * CLOCKS["sm_mhz"]
    print(json.dumps(out))


if __name__ == "__main__":
    main()
