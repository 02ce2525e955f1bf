"""Helper launched by torchrun (2+ GPUs): expert-parallel forward/backward vs the single-rank model."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist

from miles_b200.models import ParamStore, build_model, get_config
from miles_b200.parallel.expert_parallel import ExpertParallel
from miles_b200.parallel.state import init_parallel_state


def batch(cfg, lens, dev, seed):
    g = torch.Generator().manual_seed(seed)
    T = sum(lens)
    tokens = torch.randint(0, cfg.vocab_size, (T,), generator=g).to(dev).int()
    pos = torch.cat([torch.arange(l) for l in lens]).to(dev).int()
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=dev)
    rows = torch.cat([torch.arange(a + 3, a + l - 1) for a, l in zip(cu[:-1].tolist(), lens)]).to(dev)
    tg = tokens[(rows + 1).long()]
    coef = torch.randn(rows.numel(), generator=g).to(dev)
    return tokens, pos, cu, rows, tg, coef


def main():
    mode = sys.argv[1]  # nccl | fused (GEMM epilogue stores into the peers) | fused_copy (separate return kernel)
    fused = mode != "nccl"
    world = int(os.environ["WORLD_SIZE"])
    ps = init_parallel_state(ep=world)
    dev = ps.device
    cfg = get_config(sys.argv[2] if len(sys.argv) > 2 else "qwen3-smoke-moe")  # e.g. glm4moe-smoke: sigmoid router + shared expert
    lens_of = {r: [90 + 13 * r, 41, 150 - 20 * r] for r in range(world)}
    # expert-parallel model
    store = ParamStore(cfg, dev, torch.bfloat16, ep_size=world, ep_rank=ps.ep.rank, init_std=0.05, seed=5)
    store.allocate_grads(torch.float32)
    ep = ExpertParallel(cfg, ps, fused=fused, max_tokens=1024, fused_epilogue=(mode == "fused"))
    model = build_model(cfg, store, "b200", ep=ep)
    # single-rank oracle with all experts
    ref_store = ParamStore(cfg, dev, torch.bfloat16, init_std=0.05, seed=5)
    ref_store.allocate_grads(torch.float32)
    ref = build_model(cfg, ref_store, "b200")
    el = cfg.num_experts // world
    for s in store.specs:  # same global model on both layouts
        src = ref_store.params[s.name]
        if s.group == "expert":
            src = src[ps.ep.rank * el:(ps.ep.rank + 1) * el]
        assert torch.equal(store.params[s.name], src), s.name

    def loss_fn_for(coef):
        return lambda lp, ent: ((lp * coef).sum() / 40 + 0.01 * ent.sum(), {})

    for it in range(2):  # twice: the symmetric buffers and epochs are reused
        store.zero_grads()
        ref_store.zero_grads()
        tokens, pos, cu, rows, tg, coef = batch(cfg, lens_of[ps.rank], dev, 100 + ps.rank + 10 * it)
        rec = []
        lp0, _ = model.forward_logprobs(tokens, pos, cu, rows, tg, 1.0, record=rec)
        replay = torch.stack(rec, 1)
        _, _, lp, ent = model.forward_backward(tokens, pos, cu, rows, tg, 1.0, loss_fn_for(coef), replay=replay)
        model.check_status()
        ep.check_status()
        lps = {}
        for r in range(world):
            b = batch(cfg, lens_of[r], dev, 100 + r + 10 * it)
            rep_r = [torch.empty_like(replay) if r == ps.rank else None]
            # every rank needs the routing the owner of batch r recorded
            shape = torch.tensor(list(replay.shape), device=dev)
            shapes = [torch.empty_like(shape) for _ in range(world)]
            dist.all_gather(shapes, shape)
            rp = replay.clone() if r == ps.rank else torch.empty(shapes[r].tolist(), dtype=replay.dtype, device=dev)
            dist.broadcast(rp, src=r)
            _, _, lp_r, _ = ref.forward_backward(b[0], b[1], b[2], b[3], b[4], 1.0, loss_fn_for(b[5]), replay=rp)
            lps[r] = lp_r
        d = (lp - lps[ps.rank]).abs()
        assert d.max().item() < 5e-2 and d.mean().item() < 1e-2, (d.max().item(), d.mean().item())  # bf16, different reduction order
        if ps.rank == 0:
            print(f"logprob diff vs single rank: max {d.max().item():.4f} mean {d.mean().item():.5f}")
        assert torch.allclose(lp0, lp, atol=1e-5)
        # expert gradients: the owner accumulates the contributions of every rank's tokens
        for s in store.specs:
            if s.group != "expert":
                continue
            got = store.grads[s.name]
            want = ref_store.grads[s.name][ps.ep.rank * el:(ps.ep.rank + 1) * el]
            cos = torch.nn.functional.cosine_similarity(got.flatten(), want.flatten(), dim=0).item()
            assert cos > 0.995, (s.name, cos)
        # dense gradients: sum over ranks equals the oracle that saw all batches
        dense = store.grad["dense"].clone()
        dist.all_reduce(dense)
        cos = torch.nn.functional.cosine_similarity(dense, ref_store.grad["dense"], dim=0).item()
        assert cos > 0.995, cos
    if ps.rank == 0:
        print(f"EP_CHECK_OK mode={mode} world={world}")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
