"""Process groups that are destroyed and rebuilt between phases: holders all over the program get the new group without
code of their own, a non-member rank takes part in the rebuild, a collective on a released group fails loudly."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class _Holder:
    def __init__(self, group):
        self.group = group
        self.nested = {"g": group, "lst": [1, group]}


def _worker(rank: int, world: int, port: int):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    from miles_b200.parallel.reloadable_groups import RELEASED, registry
    from miles_b200.parallel.state import init_parallel_state

    ps = init_parallel_state(cp=1, backend="gloo")  # dp group over all three ranks, created through the registry
    reg = registry()
    pair = reg.new_group([0, 1])                       # rank 2 is not a member but must take part in creating it
    holder = _Holder(pair if rank < 2 else ps.dp_cp.group)
    old_dp = ps.dp_cp.group
    t = torch.ones(1) * (rank + 1)
    dist.all_reduce(t, group=ps.dp_cp.group)
    assert t.item() == 6
    n_groups_before = len(reg.records)
    reg.release(include_host_groups=True)
    assert ps.dp_cp.group is RELEASED and holder.group is RELEASED and holder.nested["lst"][1] is RELEASED
    with pytest.raises(Exception):
        dist.all_reduce(torch.ones(1), group=ps.dp_cp.group)   # fails loudly, does not fall back to the world group
    assert reg.release(include_host_groups=True) == 0          # idempotent
    got = reg.reload()
    assert got >= 1 and len(reg.records) == n_groups_before
    assert ps.dp_cp.group is not RELEASED and ps.dp_cp.group is not old_dp
    assert holder.group is holder.nested["g"] is holder.nested["lst"][1]
    t = torch.ones(1) * (rank + 1)
    dist.all_reduce(t, group=ps.dp_cp.group)
    assert t.item() == 6
    if rank < 2:
        t = torch.ones(1) * (rank + 1)
        dist.all_reduce(t, group=holder.group)
        assert t.item() == 3
    # a second cycle works the same way
    reg.release(include_host_groups=True)
    reg.reload()
    t = torch.ones(1)
    dist.all_reduce(t, group=ps.dp_cp.group)
    assert t.item() == 3
    dist.barrier()
    dist.destroy_process_group()


def test_release_and_reload_over_three_ranks():
    mp.spawn(_worker, args=(3, _free_port()), nprocs=3, join=True)


def _loop_worker(rank: int, world: int, port: int, out_dir: str):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                      MILES_B200_ENV_REPORT="0")
    torch.set_num_threads(2)
    from miles_b200.loop import RLLoop
    from miles_b200.parallel.reloadable_groups import registry
    from miles_b200.utils.arguments import parse_args

    args = parse_args(["--model-preset", "qwen3-tiny", "--rollout-batch-size", "8", "--n-samples-per-prompt", "4",
                       "--rollout-max-response-len", "16", "--rollout-max-prompt-len", "32", "--rm-type", "parity", "--lr", "1e-5",
                       "--micro-batch-size", "8", "--colocate", "--num-rollout", "2", "--actor-num-gpus-per-node", str(world),
                       "--distributed-backend", "gloo", "--reload-process-groups"])
    loop = RLLoop(args)
    first = loop.ps.dp_cp.group
    hist = loop.run()
    assert len(hist) == 2 and not registry().released
    assert loop.ps.dp_cp.group is not first, "the groups were rebuilt around every rollout"
    assert loop.actor.opt.dp_group is loop.ps.dp_cp.group, "holders follow the rebuilt group"
    flat = torch.cat([t.flatten() for t in loop.actor.store.flat.values()])
    ref = flat.clone()
    dist.broadcast(ref, src=0)
    assert torch.equal(flat, ref), "ranks stayed in step"
    dist.barrier()
    dist.destroy_process_group()


def test_training_loop_releases_groups_for_the_rollout(tmp_path):
    mp.spawn(_loop_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)


def _topo_worker(rank: int, world: int, port: int):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    from miles_b200.parallel.state import init_parallel_state
    from miles_b200.parallel.topology import group_is_single_node, peer_memory_ok

    ps = init_parallel_state(backend="gloo")
    assert group_is_single_node(ps.dp_cp.group, ps.dp_cp.size), "four local processes are one node"
    assert peer_memory_ok(ps.dp_cp.group, ps.dp_cp.size, True) and not peer_memory_ok(ps.dp_cp.group, ps.dp_cp.size, False)
    # ranks {0, 1} and {2, 3} pretend to sit on two nodes: groups inside a node keep peer memory, the group across does not
    os.environ["MILES_B200_NODE_ID"] = f"node{rank // 2}"
    from miles_b200.parallel.reloadable_groups import registry

    pairs = [registry().new_group([0, 1]), registry().new_group([2, 3])]
    across = registry().new_group([0, 1, 2, 3])
    mine = pairs[rank // 2]
    assert group_is_single_node(mine, 2)
    assert not group_is_single_node(across, 4)
    assert group_is_single_node(None, 1)
    dist.barrier()
    dist.destroy_process_group()


def test_groups_across_nodes_fall_back_from_peer_memory():
    mp.spawn(_topo_worker, args=(4, _free_port()), nprocs=4, join=True)
