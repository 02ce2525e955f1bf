#!/usr/bin/env bash
# Supervised fine-tuning on chat data through the same loop (multi-turn loss masks, no engine needed).
set -euo pipefail
NGPU=${NGPU:-8}
python -m torch.distributed.run --nnodes=1 --nproc-per-node "$NGPU" --master-addr 127.0.0.1 --master-port 29500 train.py \
  --model-preset qwen3-4B ${HF_CHECKPOINT:+--hf-checkpoint "$HF_CHECKPOINT"} --prompt-data "${PROMPT_DATA:?set PROMPT_DATA}" \
  --rollout-function-path miles_b200.rollout.sft_rollout.generate_rollout --loss-type sft_loss --debug-train-only \
  --loss-mask-type qwen3 --rollout-batch-size 128 --n-samples-per-prompt 1 --global-batch-size 128 \
  --lr 1e-5 --lr-decay-style cosine --lr-warmup-iters 10 --use-dynamic-batch-size --max-tokens-per-gpu 16384 --num-epoch 3
