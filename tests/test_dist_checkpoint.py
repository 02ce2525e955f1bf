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


@pytest.mark.parametrize("name", ["qwen3-tiny", "qwen3-tiny-moe"])
def test_hf_to_torch_dist_and_back(tmp_path, name):
    """HF safetensors -> torch_dist -> (expert-parallel slice loads it) -> HF safetensors: every tensor survives."""
    from safetensors import safe_open
    from miles_b200.checkpoint import export_hf
    from miles_b200.tools import convert_hf_to_torch_dist, convert_torch_dist_to_hf
    cfg = get_config(name)
    src = ParamStore(cfg, "cpu", torch.bfloat16, seed=21)
    one = NS(size=1, rank=0, group=None)
    actor = NS(store=src, opt=None, args=NS(hf_checkpoint=None), cfg=cfg, global_step=0, ps=NS(rank=0, world_size=1, tp=one, pp=one, dp_cp=one))
    hf0 = str(tmp_path / "hf0")
    export_hf(actor, hf0)
    d = convert_hf_to_torch_dist.convert(hf0, str(tmp_path / "dist"))
    assert dist_ckpt.is_dist_checkpoint(d)
    if cfg.is_moe:
        part = ParamStore(cfg, "cpu", torch.bfloat16, seed=3, ep_size=2, ep_rank=1)
        dist_ckpt.load(_actor(part), d, with_optimizer=False)
        want = ParamStore(cfg, "cpu", torch.bfloat16, seed=21, ep_size=2, ep_rank=1)
        for n in want.params:
            assert torch.equal(part.params[n], want.params[n]), n
    hf1 = convert_torch_dist_to_hf.convert(str(tmp_path / "dist"), str(tmp_path / "hf1"))

    def tensors(path):
        out = {}
        for f in sorted(os.listdir(path)):
            if f.endswith(".safetensors"):
                with safe_open(os.path.join(path, f), framework="pt") as h:
                    out.update({k: h.get_tensor(k) for k in h.keys()})
        return out
    a, b = tensors(hf0), tensors(hf1)
    assert a.keys() == b.keys() and len(a) > 10
    for k in a:
        assert torch.equal(a[k], b[k]), k
