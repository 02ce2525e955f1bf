"""Offline quantisation of an HF checkpoint: ``--format fp8_block | mxfp8 | nvfp4 | int4``.

Linear weights (``*_proj.weight``) are quantised; embeddings, norms, the router gate and the LM head stay in
bf16 (plus any name matching ``--ignore``).  Output tensors follow the conventions engines expect:
``<name>`` (packed values) + ``<name>_scale_inv`` (fp8 block / mxfp8) or ``<name>_scale`` +
``<name>_scale_2`` (nvfp4) or ``<name>_scale`` + ``<name>_zero_point`` (int4), and ``quantization_config``
in ``config.json``.  Runs the sm_100a quantiser kernels when a GPU is present, else the PyTorch
reference implementations.  Counterpart of tools/convert_hf_to_{fp8,mxfp8,nvfp4,int4}.py.
"""
import argparse
import json
import os
import shutil


import torch
from safetensors import safe_open
from safetensors.torch import save_file

from miles_b200.weight_sync.quantize import quantize_tensor


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--hf-checkpoint", required=True)
    ap.add_argument("--output", required=True)
    ap.add_argument("--format", required=True, choices=["fp8_block", "mxfp8", "nvfp4", "int4"])
    ap.add_argument("--ignore", nargs="*", default=["lm_head", "embed_tokens", "norm", "mlp.gate."])
    ap.add_argument("--group-size", type=int, default=32)
    a = ap.parse_args()
    os.makedirs(a.output, exist_ok=True)
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    wm = {}
    for fn in sorted(f for f in os.listdir(a.hf_checkpoint) if f.endswith(".safetensors")):
        out = {}
        with safe_open(os.path.join(a.hf_checkpoint, fn), framework="pt", device="cpu") as f:
            for name in f.keys():
                t = f.get_tensor(name)
                if t.dim() == 2 and name.endswith("_proj.weight") and not any(s in name for s in a.ignore):
                    for k, v in quantize_tensor(name, t.to(dev), a.format, group_size=a.group_size).items():
                        out[k] = v.cpu().contiguous()
                else:
                    out[name] = t
        save_file(out, os.path.join(a.output, fn), metadata={"format": "pt"})
        wm.update({k: fn for k in out})
    cfg = json.load(open(os.path.join(a.hf_checkpoint, "config.json")))
    cfg["quantization_config"] = {"quant_method": a.format, "ignore": a.ignore, "group_size": a.group_size}
    json.dump(cfg, open(os.path.join(a.output, "config.json"), "w"), indent=1)
    json.dump({"metadata": {}, "weight_map": wm}, open(os.path.join(a.output, "model.safetensors.index.json"), "w"), indent=1)
    for fn in os.listdir(a.hf_checkpoint):
        if fn.startswith("tokenizer") or fn in ("vocab.json", "merges.txt", "generation_config.json", "special_tokens_map.json"):
            shutil.copy(os.path.join(a.hf_checkpoint, fn), os.path.join(a.output, fn))


if __name__ == "__main__":
    main()
