"""Convert a HuggingFace safetensors checkpoint into the native sharded format (one file per rank).

    python -m miles_b200.tools.convert_hf_to_native --hf-checkpoint /path/to/Qwen3-4B --save /ckpt/qwen3-4b --expert-model-parallel-size 1

Writes ``<save>/iter_0000000/rank_%05d.pt`` and ``latest_checkpointed_iteration.txt`` so that
``--load <save>`` (or ``--ref-load``) starts from the converted weights.  Counterpart of the reference's
tools/convert_hf_to_torch_dist.py.
"""
import argparse
import json
import os


import torch

from miles_b200.checkpoint import LATEST, iter_dir, load_hf
from miles_b200.models import ModelConfig, ParamStore


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--hf-checkpoint", required=True)
    ap.add_argument("--save", required=True)
    ap.add_argument("--expert-model-parallel-size", type=int, default=1)
    ap.add_argument("--dtype", default="bfloat16")
    a = ap.parse_args()
    cfg = ModelConfig.from_hf_config(a.hf_checkpoint)
    d = iter_dir(a.save, 0)
    os.makedirs(d, exist_ok=True)
    for r in range(a.expert_model_parallel_size):
        store = ParamStore(cfg, "cpu", getattr(torch, a.dtype), ep_size=a.expert_model_parallel_size, ep_rank=r, init=False)
        n = load_hf(cfg, store, a.hf_checkpoint)
        torch.save({"flat": store.flat, "version": 0, "global_step": 0, "ep": (store.ep_size, r)}, os.path.join(d, f"rank_{r:05d}.pt"))
        print(f"rank {r}: {n} tensors, {store.num_local_params() / 1e9:.2f} B parameters")
    with open(os.path.join(d, "meta.json"), "w") as f:
        json.dump({"iteration": 0, "world_size": a.expert_model_parallel_size, "model": cfg.to_dict()}, f, default=str)
    with open(os.path.join(a.save, LATEST), "w") as f:
        f.write("0")


if __name__ == "__main__":
    main()
