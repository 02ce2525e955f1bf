#!/usr/bin/env bash
# Prefill / decode disaggregation: the trainer (GPUs 0-1) launches the engines of pd_disaggregation.yaml on the GPUs
# after its own (two prefill engines, four decode engines), generates through them and broadcasts weight updates to all.
set -euo pipefail
HERE="$(cd "$(dirname "$0")" && pwd)"
TRAIN=${TRAIN:-2}
python -m torch.distributed.run --nnodes=1 --nproc-per-node "$TRAIN" --master-addr 127.0.0.1 --master-port 29500 train.py \
  --model-preset qwen3-4B ${HF_CHECKPOINT:+--hf-checkpoint "$HF_CHECKPOINT"} ${PROMPT_DATA:+--prompt-data "$PROMPT_DATA"} \
  --launch-rollout-fleet --sglang-config "$HERE/pd_disaggregation.yaml" \
  --num-rollout 100 --rollout-batch-size 64 --n-samples-per-prompt 8 --rollout-max-prompt-len 4096 --rollout-max-response-len 2048 \
  --rm-type deepscaler --advantage-estimator grpo --use-tis --lr 1e-6 --use-dynamic-batch-size --max-tokens-per-gpu 32768 \
  --actor-num-nodes 1 --actor-num-gpus-per-node "$TRAIN"
