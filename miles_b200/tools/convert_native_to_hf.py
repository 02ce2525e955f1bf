"""Convert a native checkpoint (all ranks) into HuggingFace safetensors shards.

    python -m miles_b200.tools.convert_native_to_hf --load /ckpt/run --ckpt-step 10 --output /export/hf

Counterpart of the reference's tools/convert_torch_dist_to_hf.py.
"""
import argparse
import json
import os


import torch
from safetensors.torch import save_file

from miles_b200.checkpoint import iter_dir, latest_iteration
from miles_b200.models import ModelConfig, ParamStore
from miles_b200.models.hf_mapping import hf_names


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--load", required=True)
    ap.add_argument("--ckpt-step", type=int, default=None)
    ap.add_argument("--output", required=True)
    ap.add_argument("--max-shard-gb", type=float, default=5.0)
    a = ap.parse_args()
    it = a.ckpt_step if a.ckpt_step is not None else latest_iteration(a.load)
    d = iter_dir(a.load, it)
    meta = json.load(open(os.path.join(d, "meta.json")))
    cfg = ModelConfig(**{k: v for k, v in meta["model"].items() if k in ModelConfig.__dataclass_fields__})
    ranks = sorted(f for f in os.listdir(d) if f.startswith("rank_"))
    os.makedirs(a.output, exist_ok=True)
    shards, cur, size, limit = [], {}, 0, int(a.max_shard_gb * (1 << 30))
    for ri, fn in enumerate(ranks):
        state = torch.load(os.path.join(d, fn), map_location="cpu", weights_only=False)
        ep_size, ep_rank = state.get("ep", (1, 0))
        store = ParamStore(cfg, "cpu", next(iter(state["flat"].values())).dtype, ep_size=ep_size, ep_rank=ep_rank, init=False)
        for g, t in state["flat"].items():
            store.flat[g].copy_(t)
        for name, t in hf_names(cfg, store):
            if ".experts." not in name and ri > 0:
                continue
            nb = t.numel() * t.element_size()
            if cur and size + nb > limit:
                shards.append(cur)
                cur, size = {}, 0
            cur[name] = t.clone().contiguous()
            size += nb
    if cur:
        shards.append(cur)
    wm = {}
    for i, sh in enumerate(shards):
        fn = f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
        save_file(sh, os.path.join(a.output, fn), metadata={"format": "pt"})
        wm.update({k: fn for k in sh})
    json.dump({"metadata": {}, "weight_map": wm}, open(os.path.join(a.output, "model.safetensors.index.json"), "w"), indent=1)
    json.dump(cfg.to_hf_config(), open(os.path.join(a.output, "config.json"), "w"), indent=1)
    open(os.path.join(a.output, ".complete"), "w").write("ok")
    print(f"wrote {len(wm)} tensors in {len(shards)} shards to {a.output}")


if __name__ == "__main__":
    main()
