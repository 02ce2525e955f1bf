"""Helper launched by torchrun (2 GPUs): a context-parallel training step on the sm_100a model path (all-to-all layout:
sequence shards are traded for head shards around the attention kernels, forward and backward) against the same step on
one rank: log-probs of the local rows and the summed gradients."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist

from miles_b200.models import ParamStore, build_model, get_config
from miles_b200.parallel.context_parallel import local_index_map, segments, zigzag_positions, zigzag_slice
from miles_b200.parallel.state import init_parallel_state


def main():
    world = int(os.environ["WORLD_SIZE"])
    ps = init_parallel_state(cp=world)
    dev, rank = ps.device, ps.cp.rank
    for preset in ("qwen3-smoke", "qwen3-smoke-moe"):
        cfg = get_config(preset)
        lens = [700, 129, 1500]
        T = sum(lens)
        g = torch.Generator().manual_seed(11)
        tokens = torch.randint(0, cfg.vocab_size, (T,), generator=g).int()
        pos = torch.cat([torch.arange(n) for n in lens]).int()
        cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
        rows = torch.cat([torch.arange(a + 5, a + n - 1) for a, n in zip(cu[:-1].tolist(), lens)])
        targets = tokens[(rows + 1).long()]
        coef = torch.randn(rows.numel(), generator=g)
        denom = float(rows.numel())

        def loss_for(c):
            return lambda lp, ent: ((lp * c).sum() / denom + 0.01 * ent.sum() / denom, {})

        # one rank, whole batch
        ref_store = ParamStore(cfg, dev, torch.bfloat16, init_std=0.05, seed=5)
        ref_store.allocate_grads(torch.float32)
        ref = build_model(cfg, ref_store, "b200")
        rec = []
        ref.forward_logprobs(tokens.to(dev), pos.to(dev), cu.to(dev), rows.to(dev), targets.to(dev), 1.0, record=rec)
        replay = torch.stack(rec, 1) if rec else None
        _, _, lp_ref, _ = ref.forward_backward(tokens.to(dev), pos.to(dev), cu.to(dev), rows.to(dev), targets.to(dev), 1.0,
                                               loss_for(coef.to(dev)), replay=replay)
        # this rank's zigzag shard
        store = ParamStore(cfg, dev, torch.bfloat16, init_std=0.05, seed=5)
        store.allocate_grads(torch.float32)
        model = build_model(cfg, store, "b200")
        lmap = local_index_map(lens, world, rank)
        loc = lmap[rows]
        keep = loc >= 0
        local_lens = [sum(b - a for a, b in segs) for segs in segments(lens, world, rank)]
        cu_l = torch.tensor([0] + list(torch.tensor(local_lens).cumsum(0)), dtype=torch.int32)
        model.cp_ctx = (lens, world, rank, ps.cp.group, "a2a", "zigzag")
        rp = zigzag_slice(replay, lens, world, rank).contiguous() if replay is not None else None
        _, _, lp, _ = model.forward_backward(zigzag_slice(tokens, lens, world, rank).to(dev), zigzag_positions(lens, world, rank).int().to(dev),
                                             cu_l.to(dev), loc[keep].to(dev), targets[keep].to(dev), 1.0, loss_for(coef[keep].to(dev)),
                                             replay=rp)
        model.check_status()
        d = (lp - lp_ref[keep.to(dev)]).abs()
        assert d.max().item() < 6e-2 and d.mean().item() < 1e-2, (preset, d.max().item(), d.mean().item())
        for grp in ("dense", "expert"):
            gl = store.grad[grp]
            if gl is None or gl.numel() == 0:
                continue
            gl = gl.clone()
            dist.all_reduce(gl, group=ps.cp.group)
            cos = torch.nn.functional.cosine_similarity(gl.float(), ref_store.grad[grp].float(), dim=0).item()
            rel = ((gl.float() - ref_store.grad[grp].float()).norm() / ref_store.grad[grp].float().norm()).item()
            assert cos > 0.995 and rel < 0.12, (preset, grp, cos, rel)
        if ps.rank == 0:
            print(f"cp train {preset}: logprob diff max {d.max().item():.4f} mean {d.mean().item():.5f}", flush=True)
        dist.barrier()
    if ps.rank == 0:
        print(f"CP_TRAIN_CHECK_OK world={world}")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
