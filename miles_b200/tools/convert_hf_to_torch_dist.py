"""Convert a HuggingFace safetensors checkpoint into the reshardable ``torch_dist`` checkpoint format.

    python -m miles_b200.tools.convert_hf_to_torch_dist --hf-checkpoint /path/to/Qwen3-30B-A3B --save /ckpt/qwen3-30b-a3b
    torchrun --nproc-per-node 8 --master-addr 127.0.0.1 -m miles_b200.tools.convert_hf_to_torch_dist ...   # experts split over 8 writers

Writes ``<save>/iter_0000000/`` (``.metadata``, ``__*.distcp``, ``meta.json``) and ``latest_checkpointed_iteration.txt``,
so ``--load <save>`` or ``--ref-load <save>`` starts from the converted weights under any tensor- / expert- / pipeline-
parallel layout. Under ``torchrun`` every process converts one expert-parallel slice (gloo, CPU only), which bounds the
host memory per process at (dense + experts / world). Counterpart of the reference's tools/convert_hf_to_torch_dist.py.
"""
import argparse
import os
from types import SimpleNamespace as NS

import torch
import torch.distributed as dist

from miles_b200.checkpoint import LATEST, dist_ckpt, iter_dir, load_hf
from miles_b200.models import ModelConfig, ParamStore


def convert(hf_checkpoint: str, save: str, dtype: torch.dtype = torch.bfloat16, iteration: int = 0) -> str:
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("gloo")
    cfg = ModelConfig.from_hf_config(hf_checkpoint)
    ep = world if (cfg.is_moe and cfg.num_experts % world == 0) else 1
    assert ep == world or world == 1, f"{world} writers need a mixture-of-experts model whose expert count divides by {world}"
    store = ParamStore(cfg, "cpu", dtype, ep_size=ep, ep_rank=rank if ep > 1 else 0, init=False)
    n = load_hf(cfg, store, hf_checkpoint)
    d = iter_dir(save, iteration)
    actor = NS(store=store, opt=None, args=NS(no_save_optim=True), ps=NS(rank=rank, world_size=world), cfg=cfg, global_step=0)
    dist_ckpt.save(actor, d, iteration)
    if world > 1:
        dist.barrier()
    if rank == 0:
        with open(os.path.join(save, LATEST), "w") as f:
            f.write(str(iteration))
    print(f"rank {rank}: {n} tensors, {store.num_local_params() / 1e9:.3f} B parameters -> {d}", flush=True)
    return d


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--hf-checkpoint", required=True)
    ap.add_argument("--save", required=True)
    ap.add_argument("--dtype", default="bfloat16")
    a = ap.parse_args()
    convert(a.hf_checkpoint, a.save, getattr(torch, a.dtype))
    if dist.is_initialized():
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
