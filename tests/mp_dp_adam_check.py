"""Helper launched by torchrun (2 GPUs): partitioned optimizer over peer memory vs all-reduce + replicated Adam."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist

from miles_b200.models import ParamStore, get_config
from miles_b200.parallel.dp_optimizer import ShardedDenseAdam
from miles_b200.parallel.state import init_parallel_state
from miles_b200.trainer.optimizer import FlatAdam, OptimConfig


def main():
    world = int(os.environ["WORLD_SIZE"])
    ps = init_parallel_state()
    dev = ps.device
    cfg = get_config("qwen3-smoke")
    oc = OptimConfig(lr=1e-3, weight_decay=0.1, clip_grad=1.0, master_weights=True)
    a = ParamStore(cfg, dev, torch.bfloat16, seed=3)
    a.allocate_grads(torch.float32)
    b = ParamStore(cfg, dev, torch.bfloat16, seed=3)
    b.allocate_grads(torch.float32)
    shard = ShardedDenseAdam(a, ps.dp_cp.group, ps.dp_cp.rank, world, dev, oc)
    assert a.grad["dense"].data_ptr() == shard.grad_sym.data_ptr() and a.params["embed.weight"].data_ptr() == shard.param_sym.data_ptr()
    opt_a = FlatAdam(a, oc, dp_group=ps.dp_cp.group, dense_shard=shard)
    opt_b = FlatAdam(b, oc, dp_group=ps.dp_cp.group)
    gen = torch.Generator(device=dev).manual_seed(100 + ps.rank)
    for it in range(3):
        g = torch.randn(a.grad["dense"].shape, generator=gen, device=dev) * 0.01
        a.grad["dense"].copy_(g)
        b.grad["dense"].copy_(g)
        dist.all_reduce(b.grad["dense"])  # the baseline: all-reduce, then every rank updates everything
        na = opt_a.step(1.0)
        nb = opt_b.step(1.0)
        shard.check_status()
        assert abs(float(na) - float(nb)) / float(nb) < 1e-4, (float(na), float(nb))
        pa, pb = a.flat["dense"].float(), b.flat["dense"].float()
        assert (pa - pb).abs().max().item() <= 2e-3 * pb.abs().max().item(), (pa - pb).abs().max().item()
        assert (pa != pb).float().mean().item() < 1e-3  # bf16 results agree except for rare rounding ties
        both = [torch.empty_like(a.flat["dense"]) for _ in range(world)]
        dist.all_gather(both, a.flat["dense"])
        assert all(torch.equal(both[0], t) for t in both), "ranks hold different parameters after the push"
    assert shard.m.numel() < a.flat["dense"].numel()  # states only for the owned range
    if ps.rank == 0:
        print(f"DP_ADAM_CHECK_OK world={world} shard={shard.hi - shard.lo} of {a.flat['dense'].numel()}")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
