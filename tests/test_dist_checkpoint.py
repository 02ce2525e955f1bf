"""Reshardable checkpoints (torch.distributed.checkpoint format): what one parallel layout saves, another loads."""
import os
import socket
from types import SimpleNamespace as NS

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from miles_b200.checkpoint import dist_ckpt
from miles_b200.models import ParamStore, get_config


def _actor(store, rank=0, world=1):
    return NS(store=store, opt=None, args=NS(no_save_optim=True), ps=NS(rank=rank, world_size=world), cfg=store.global_cfg,
              global_step=3)


def _save_worker(rank, world, port, out, kind):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    if kind == "tp":
        store = ParamStore(get_config("qwen3-tiny"), "cpu", torch.float32, seed=9, tp_size=world, tp_rank=rank)
    else:
        store = ParamStore(get_config("qwen3-tiny-moe"), "cpu", torch.float32, seed=9, ep_size=world, ep_rank=rank)
    dist_ckpt.save(_actor(store, rank, world), out, 7)
    dist.barrier()
    dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("kind", ["tp", "ep"])
def test_checkpoint_saved_by_two_ranks_loads_on_one(tmp_path, kind):
    """Two tensor-parallel (or expert-parallel) ranks save their shards; a single-rank layout loads the whole model,
    and a differently sharded single rank (the other half) loads just its part."""
    out = str(tmp_path / "ck")
    mp.spawn(_save_worker, args=(2, _free_port(), out, kind), nprocs=2, join=True)
    assert dist_ckpt.is_dist_checkpoint(out)
    name = "qwen3-tiny" if kind == "tp" else "qwen3-tiny-moe"
    want = ParamStore(get_config(name), "cpu", torch.float32, seed=9)            # the model the shards were cut from
    got = ParamStore(get_config(name), "cpu", torch.float32, seed=1234)          # other weights: everything must be overwritten
    meta = dist_ckpt.load(_actor(got), out, with_optimizer=False)
    assert meta["rollout_id"] == 7 and meta["saved_layout"][kind] == 2
    for n in want.params:
        assert torch.equal(got.params[n], want.params[n]), n
    kw = dict(tp_size=2, tp_rank=1) if kind == "tp" else dict(ep_size=2, ep_rank=1)
    part_want = ParamStore(get_config(name), "cpu", torch.float32, seed=9, **kw)
    part = ParamStore(get_config(name), "cpu", torch.float32, seed=77, **kw)
    dist_ckpt.load(_actor(part), out, with_optimizer=False)
    for n in part_want.params:
        assert torch.equal(part.params[n], part_want.params[n]), n


def test_missing_atoms_are_reported(tmp_path):
    out = str(tmp_path / "ck")
    small = ParamStore(get_config("qwen3-tiny"), "cpu", torch.float32, seed=1, pp_size=2, pp_rank=0)   # first stage only
    dist_ckpt.save(_actor(small), out, 0)
    full = ParamStore(get_config("qwen3-tiny"), "cpu", torch.float32, seed=2)
    with pytest.raises(KeyError, match="lacks"):
        dist_ckpt.load(_actor(full), out, with_optimizer=False)
