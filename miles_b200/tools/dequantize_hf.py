"""Cast a quantised HF checkpoint back to bf16: ``fp8_block | mxfp8 | nvfp4 | int4`` (read from ``quantization_config``
in ``config.json``, or ``--format``).

    python -m miles_b200.tools.dequantize_hf --hf-checkpoint /ckpt/q --output /ckpt/bf16

Every ``<name>`` that has companion scale tensors (``<name>_scale_inv``; ``<name>_scale`` + ``<name>_scale_2``;
``<name>_scale`` + ``<name>_zero_point``) is multiplied out to bf16 and the companions are dropped; everything else is
copied. Counterpart of the reference's tools/fp8_cast_bf16.py and tools/convert_kimi_int4_to_bf16.py, for the formats
``quantize_hf`` writes.
"""
import argparse
import json
import os
import shutil

import torch
from safetensors import safe_open
from safetensors.torch import save_file

from miles_b200.ops import reference as R

_COMPANIONS = ("_scale_inv", "_scale_2", "_scale", "_zero_point")


def dequantize(fmt: str, name: str, tensors: dict, group_size: int = 32) -> torch.Tensor:
    q = tensors[name]
    if fmt == "fp8_block":
        s = tensors[name + "_scale_inv"].float()
        rows, cols = q.shape
        full = s.repeat_interleave(128, 0).repeat_interleave(128, 1)[:rows, :cols]
        return (q.float() * full).to(torch.bfloat16)
    if fmt == "mxfp8":
        return R.mxfp8_dequant(q.view(torch.float8_e4m3fn) if q.dtype == torch.uint8 else q, tensors[name + "_scale_inv"]).to(torch.bfloat16)
    if fmt == "nvfp4":
        packed = q.view(torch.uint8)
        code = torch.stack([packed & 0xF, packed >> 4], -1).reshape(*packed.shape[:-1], packed.shape[-1] * 2)
        sf = tensors[name + "_scale"]
        sf = sf.view(torch.float8_e4m3fn) if sf.dtype == torch.uint8 else sf
        return R.nvfp4_dequant(code, sf, tensors[name + "_scale_2"].float().reshape(())).to(torch.bfloat16)
    if fmt == "int4":
        s, z = tensors[name + "_scale"].float(), tensors[name + "_zero_point"].float()
        rows, cols = q.shape
        g = cols // s.shape[-1]
        return ((q.float().reshape(rows, cols // g, g) - z.reshape(rows, -1, 1)) * s.reshape(rows, -1, 1)).reshape(rows, cols).to(torch.bfloat16)
    raise ValueError(f"unknown quantisation format {fmt!r}")


def convert(hf_checkpoint: str, output: str, fmt: str = None) -> int:
    cfg = json.load(open(os.path.join(hf_checkpoint, "config.json")))
    qc = cfg.pop("quantization_config", None) or {}
    fmt = fmt or qc.get("quant_method")
    assert fmt, "the checkpoint has no quantization_config: pass --format"
    os.makedirs(output, exist_ok=True)
    wm, n = {}, 0
    for fn in sorted(f for f in os.listdir(hf_checkpoint) if f.endswith(".safetensors")):
        with safe_open(os.path.join(hf_checkpoint, fn), framework="pt", device="cpu") as f:
            tensors = {k: f.get_tensor(k) for k in f.keys()}
        out = {}
        for name, t in tensors.items():
            base = next((name[:-len(c)] for c in _COMPANIONS if name.endswith(c) and name[:-len(c)] in tensors), None)
            if base is not None:
                continue  # a companion of a quantised tensor
            if any((name + c) in tensors for c in _COMPANIONS):
                out[name] = dequantize(fmt, name, tensors, qc.get("group_size", 32)).contiguous()
                n += 1
            else:
                out[name] = t
        save_file(out, os.path.join(output, fn), metadata={"format": "pt"})
        wm.update({k: fn for k in out})
    json.dump(cfg, open(os.path.join(output, "config.json"), "w"), indent=1)
    json.dump({"metadata": {}, "weight_map": wm}, open(os.path.join(output, "model.safetensors.index.json"), "w"), indent=1)
    for fn in os.listdir(hf_checkpoint):
        if fn.startswith("tokenizer") or fn in ("vocab.json", "merges.txt", "generation_config.json", "special_tokens_map.json"):
            shutil.copy(os.path.join(hf_checkpoint, fn), os.path.join(output, fn))
    return n


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--hf-checkpoint", required=True)
    ap.add_argument("--output", required=True)
    ap.add_argument("--format", default=None, choices=[None, "fp8_block", "mxfp8", "nvfp4", "int4"])
    a = ap.parse_args()
    print(f"dequantised {convert(a.hf_checkpoint, a.output, a.format)} tensors into {a.output}")


if __name__ == "__main__":
    main()
