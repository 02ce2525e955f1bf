"""Convert a ``torch_dist`` checkpoint (any parallel layout) into HuggingFace safetensors shards.

    python -m miles_b200.tools.convert_torch_dist_to_hf --load /ckpt/run --ckpt-step 10 --output /export/hf [--hf-checkpoint /orig]

Reads the model shape from the checkpoint's ``meta.json``, loads the weights into one host copy (optimizer state is not
read), writes ``model-XXXXX-of-YYYYY.safetensors`` + index + ``config.json`` and copies the tokenizer files of
``--hf-checkpoint`` when given. Counterpart of the reference's tools/convert_torch_dist_to_hf.py.
"""
import argparse
import json
import os
from types import SimpleNamespace as NS

import torch

from miles_b200.checkpoint import dist_ckpt, export_hf, iter_dir, latest_iteration
from miles_b200.models import ModelConfig, ParamStore


def convert(load: str, output: str, ckpt_step=None, hf_checkpoint=None, dtype: torch.dtype = torch.bfloat16,
            max_shard_gb: float = 5.0) -> str:
    it = ckpt_step if ckpt_step is not None else latest_iteration(load)
    d = iter_dir(load, it) if it is not None else load
    assert dist_ckpt.is_dist_checkpoint(d), f"{d} is not a torch_dist checkpoint (no .metadata); use convert_native_to_hf for the per-rank format"
    meta = json.load(open(os.path.join(d, "meta.json")))
    cfg = ModelConfig(**{k: v for k, v in meta["model"].items() if k in ModelConfig.__dataclass_fields__})
    store = ParamStore(cfg, "cpu", dtype, init=False)
    one = NS(size=1, rank=0, group=None)
    actor = NS(store=store, opt=None, args=NS(no_save_optim=True, hf_checkpoint=hf_checkpoint), cfg=cfg, global_step=0,
               ps=NS(rank=0, world_size=1, tp=one, pp=one, dp_cp=one))
    dist_ckpt.load(actor, d, with_optimizer=False)
    export_hf(actor, output, max_shard_bytes=int(max_shard_gb * (1 << 30)), tokenizer_dir=hf_checkpoint)
    return output


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--load", required=True)
    ap.add_argument("--ckpt-step", type=int, default=None)
    ap.add_argument("--output", required=True)
    ap.add_argument("--hf-checkpoint", default=None, help="copy tokenizer files from here")
    ap.add_argument("--dtype", default="bfloat16")
    ap.add_argument("--max-shard-gb", type=float, default=5.0)
    a = ap.parse_args()
    out = convert(a.load, a.output, a.ckpt_step, a.hf_checkpoint, getattr(torch, a.dtype), a.max_shard_gb)
    print(f"wrote {out}")


if __name__ == "__main__":
    main()
