"""Helper launched by torchrun (2+ GPUs): the low-latency expert-parallel decode exchange.

1. one MoE layer through ``EpDecodeLL.moe_decode`` against the single-rank layer on a full copy of the experts, with a
   different number of rows on every rank, padding rows, and several rounds over the same buffers (epochs);
2. whole rollouts through a lockstep engine (ranks hold different numbers of requests of different lengths, so ranks
   run padding-only steps while others still decode), checked by recomputing the log-probs of what was generated with
   the single-rank model under routing replay;
3. ``timing``: microseconds per MoE layer of the exchange path for a few row counts (CUDA events, max over ranks).
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist

from miles_b200.engine import Engine, SamplingParams
from miles_b200.engine.core import LockstepSync
from miles_b200.models import ParamStore, build_model, get_config
from miles_b200.parallel.ep_decode import EpDecodeLL
from miles_b200.parallel.expert_parallel import ExpertParallel
from miles_b200.parallel.state import init_parallel_state


def layer_check(cfg, ps, model, ref, ll, dev):
    C = model.C
    world = ps.world_size
    i = next(j for j in range(cfg.num_layers) if cfg.layer_is_moe(j))
    p = f"layers.{i}."
    for rnd, bound in enumerate((8, 8, 16, 2, 64)):
        T = max(1, min(bound, (3 + 5 * ps.rank + 7 * rnd) % (bound + 1)))
        g = torch.Generator(device=dev).manual_seed(1000 * rnd + ps.rank)
        x2 = (torch.randn(T, cfg.hidden_size, device=dev, generator=g) * 0.5).bfloat16()
        active = torch.ones(bound, dtype=torch.int32, device=dev)
        if T > 1:
            active[T - 1] = 0  # a padding row: must come back as the residual, and cost no expert work
        ll.set_step(bound, active)
        h2 = None
        if T > 8:
            h2, _ = C.rmsnorm_fwd(x2, None, ref.store.params[p + "ln2.weight"], cfg.rms_eps)
        rec = []
        y = ll.moe_decode(model, i, x2, h2, rec)
        ll.check_status()
        model.check_status()
        hh, _ = C.rmsnorm_fwd(x2, None, ref.store.params[p + "ln2.weight"], cfg.rms_eps)
        rec_ref = []
        want, _ = ref.moe_forward(i, hh, None, rec_ref, keep=False, residual=x2)
        assert torch.equal(rec[0][:T], rec_ref[0][:T]), "router picks differ from the single-rank router"
        live = active[:T].bool()
        err = (y[live].float() - want[live].float()).abs().max().item() / (want[live].float().abs().max().item() + 1e-6)
        assert err < 2e-2, (rnd, T, err)
        if (~live).any():
            assert torch.equal(y[~live], x2[~live]), "a padding row must pass through unchanged"
    dist.barrier()


def rollout_check(cfg, ps, store, model, ref, ll, dev, use_graph=True, overlap=True, report=False):
    world = ps.world_size
    sync = LockstepSync(ps.gloo_world)
    eng = Engine(model, sync=sync, ep_decode=ll, max_running=8, page_size=64, max_seq_len=512, use_cuda_graph=use_graph)
    eng.overlap_decode = overlap
    eng.warm_up_decode_graphs()
    g = torch.Generator().manual_seed(50 + ps.rank)
    n_req = 5 if ps.rank == 0 else 2
    prompts = [torch.randint(0, cfg.vocab_size, (20 + 9 * j + 3 * ps.rank,), generator=g).tolist() for j in range(n_req)]
    params = [SamplingParams(temperature=1.0, max_new_tokens=96, forced_length=12 + 11 * j + 20 * (ps.rank == 0), ignore_eos=True,
                             sampling_seed=7 + j) for j in range(n_req)]
    res = eng.generate(prompts, params, return_routed_experts=True)
    eng.drain()
    ll.check_status()
    model.check_status()
    toks, pos, rows, tgts, cu, routes, lps = [], [], [], [], [0], [], []
    for pr, sp, r in zip(prompts, params, res):
        out = r["output_ids"]
        assert len(out) == sp.forced_length, (len(out), sp.forced_length)
        ids = pr + out
        re = r["meta_info"]["routed_experts"].to(torch.int32)
        routes.append(torch.cat([re, re[-1:].expand(len(ids) - re.shape[0], -1, -1)], 0))
        rows += list(range(cu[-1] + len(pr) - 1, cu[-1] + len(ids) - 1))
        tgts += out
        toks += ids
        pos += list(range(len(ids)))
        cu.append(cu[-1] + len(ids))
        lps += [lp for lp, _ in r["meta_info"]["output_token_logprobs"]]
    t = lambda v, dt=torch.int32: torch.tensor(v, dtype=dt, device=dev)
    lp_ref, _ = ref.forward_logprobs(t(toks), t(pos), t(cu), t(rows, torch.int64), t(tgts), 1.0,
                                     replay=torch.cat(routes).contiguous().to(dev))
    diff = (lp_ref - torch.tensor(lps, device=dev)).abs()
    if report:
        first = torch.tensor([sum(len(r["output_ids"]) for r in res[:j]) for j in range(len(res))], device=dev)
        per_req = [round(float(diff[a:a + len(r["output_ids"])].mean()), 4) for a, r in zip(first.tolist(), res)]
        worst = int(diff.argmax())
        print(f"[rank {ps.rank}] graph={use_graph} overlap={overlap} ll={getattr(ll, 'low_latency', False)} mean={diff.mean().item():.4f} "
              f"max={diff.max().item():.3f} at flat index {worst} first-token mean={diff[first].mean().item():.4f} per-request={per_req} "
              f"lens={[len(r['output_ids']) for r in res]}", flush=True)
        dist.barrier()
        return diff.mean().item(), 0
    assert diff.mean().item() < 2e-2 and diff.max().item() < 0.3, (diff.mean().item(), diff.max().item())
    steps = torch.tensor([eng.stats["decode_steps"]], device=dev)
    dist.all_reduce(steps, op=dist.ReduceOp.MAX)
    dist.barrier()
    return diff.mean().item(), int(steps.item())


def timing(cfg, ps, model, ll, dev, layers=48, iters=20):
    i = next(j for j in range(cfg.num_layers) if cfg.layer_is_moe(j))
    out = {}
    for T in (1, 8, 32, 64):
        x2 = (torch.randn(T, cfg.hidden_size, device=dev) * 0.5).bfloat16()
        active = torch.ones(T, dtype=torch.int32, device=dev)
        ll.set_step(T, active)
        h2 = None
        if T > 8:
            h2, _ = model.C.rmsnorm_fwd(x2, None, model.store.params[f"layers.{i}.ln2.weight"], cfg.rms_eps)

        def body():
            y = x2
            for _ in range(layers):
                y = ll.moe_decode(model, i, x2, h2, None)
            return y

        body()
        torch.cuda.synchronize()
        dist.barrier()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            body()
        dist.barrier()
        for _ in range(3):
            gr.replay()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            gr.replay()
        e1.record()
        torch.cuda.synchronize()
        us = torch.tensor([e0.elapsed_time(e1) * 1e3 / (iters * layers)], device=dev)
        dist.all_reduce(us, op=dist.ReduceOp.MAX)
        out[T] = float(us.item())
        ll.check_status()
    return out


def main():
    mode = sys.argv[1] if len(sys.argv) > 1 else "check"
    preset = sys.argv[2] if len(sys.argv) > 2 else "qwen3-smoke-moe"
    world = int(os.environ["WORLD_SIZE"])
    ps = init_parallel_state(ep=world)
    dev = ps.device
    cfg = get_config(preset)
    if mode == "timing" and preset != "qwen3-smoke-moe":
        import copy

        cfg = copy.copy(cfg)
        cfg.num_layers = 2  # real layer shapes, two layers' worth of weights
    store = ParamStore(cfg, dev, torch.bfloat16, ep_size=world, ep_rank=ps.ep.rank, init_std=0.05, seed=5)
    ep = ExpertParallel(cfg, ps, fused=True, max_tokens=1024)
    model = build_model(cfg, store, "b200", ep=ep)
    ll = EpDecodeLL(cfg, ps, max_rows=64, wait_ms=2000.0)
    if mode == "timing":
        us = timing(cfg, ps, model, ll, dev)
        if ps.rank == 0:
            print("EP_DECODE_TIMING " + " ".join(f"T={t}:{v:.1f}us" for t, v in us.items()) + f" world={world} model={preset}")
    else:
        ref_store = ParamStore(cfg, dev, torch.bfloat16, init_std=0.05, seed=5)
        ref = build_model(cfg, ref_store, "b200")
        layer_check(cfg, ps, model, ref, ll, dev)
        if mode == "diagnose":
            for kw in (dict(use_graph=True, overlap=True), dict(use_graph=False, overlap=False), dict(use_graph=False, overlap=True),
                       dict(use_graph=True, overlap=False)):
                rollout_check(cfg, ps, store, model, ref, ll, dev, report=True, **kw)
            rollout_check(cfg, ps, store, model, ref, ep, dev, report=True, use_graph=False, overlap=False)
            dist.barrier()
            dist.destroy_process_group()
            return
        mean_diff, steps = rollout_check(cfg, ps, store, model, ref, ll, dev)
        if ps.rank == 0:
            print(f"EP_DECODE_CHECK_OK world={world} logprob_diff={mean_diff:.5f} lockstep_decode_steps={steps}")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
