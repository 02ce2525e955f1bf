#!/usr/bin/env bash
# Checkpoint conversions around a run (reference: tools/convert_hf_to_torch_dist.py, convert_torch_dist_to_hf.py,
# convert_hf_to_{fp8,mxfp8,nvfp4,int4}.py, fp8_cast_bf16.py).
set -euo pipefail
HF=${HF_CHECKPOINT:?path of a HuggingFace checkpoint}
OUT=${OUT:-/tmp/miles_b200_ckpt}
# HF safetensors -> reshardable torch_dist checkpoint (use as --load / --ref-load under any TP / EP / PP layout);
# under torchrun every process converts one expert-parallel slice
python -m miles_b200.tools.convert_hf_to_torch_dist --hf-checkpoint "$HF" --save "$OUT/dist"
# ... train with --load "$OUT/dist" --save "$OUT/run" --save-interval 20 [--async-save] ...
# a saved iteration -> HF safetensors (tokenizer files copied from the original)
python -m miles_b200.tools.convert_torch_dist_to_hf --load "$OUT/dist" --output "$OUT/hf" --hf-checkpoint "$HF"
# offline quantisation for serving, and back to bf16
python -m miles_b200.tools.quantize_hf --hf-checkpoint "$OUT/hf" --output "$OUT/hf-mxfp8" --format mxfp8
python -m miles_b200.tools.dequantize_hf --hf-checkpoint "$OUT/hf-mxfp8" --output "$OUT/hf-bf16"
