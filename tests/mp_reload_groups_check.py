"""Helper launched by torchrun (2+ GPUs): NCCL sub-groups are destroyed and rebuilt (parallel/reloadable_groups.py). Prints
the device memory that the release gave back and checks that collectives work on the rebuilt groups, that an optimizer
holding a group follows the rebuild, and that a second cycle works."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist

from miles_b200.parallel.reloadable_groups import RELEASED, registry
from miles_b200.parallel.state import init_parallel_state


class Holder:
    def __init__(self, g):
        self.group = g


def main():
    ps = init_parallel_state()
    dev, rank, world = ps.device, ps.rank, ps.world_size
    reg = registry()
    extra = [reg.new_group(list(range(world))) for _ in range(3)]
    holders = [Holder(g) for g in extra] + [Holder(ps.dp_cp.group)]
    x = torch.ones(1 << 20, device=dev)
    for h in holders:  # communicators are created on first use
        dist.all_reduce(x, group=h.group)
    torch.cuda.synchronize()
    assert float(x[0]) == float(world) ** len(holders)
    for cycle in range(2):
        free0 = torch.cuda.mem_get_info(dev)[0]
        freed = reg.release()
        assert all(h.group is RELEASED for h in holders)
        free1 = torch.cuda.mem_get_info(dev)[0]
        n = reg.reload()
        assert n >= len(holders) and all(h.group is not RELEASED for h in holders)
        y = torch.ones(1 << 20, device=dev)
        for h in holders:
            dist.all_reduce(y, group=h.group)
        torch.cuda.synchronize()
        assert float(y[0]) == float(world) ** len(holders)
        if rank == 0:
            print(f"cycle {cycle}: release() returned {freed / 2**20:.1f} MiB, free memory {free0 / 2**20:.0f} -> {free1 / 2**20:.0f} MiB "
                  f"with {len(holders)} groups of {world} ranks down", flush=True)
    dist.barrier()
    if rank == 0:
        print(f"RELOAD_GROUPS_OK world={world}")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
