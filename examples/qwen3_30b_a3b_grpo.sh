#!/usr/bin/env bash
# Qwen3-30B-A3B GRPO on one node (reference recipe: scripts/run_qwen3_30b_a3b.py). NGPU in {1, 2, 4, 8}.
set -euo pipefail
NGPU=${NGPU:-8}
python -m torch.distributed.run --nnodes=1 --nproc-per-node "$NGPU" --master-addr 127.0.0.1 --master-port 29500 train.py \
  --model-preset qwen3-30B-A3B ${HF_CHECKPOINT:+--hf-checkpoint "$HF_CHECKPOINT"} ${PROMPT_DATA:+--prompt-data "$PROMPT_DATA"} \
  --num-rollout 100 --rollout-batch-size $((8 * NGPU)) --n-samples-per-prompt 8 \
  --rollout-max-prompt-len 1024 --rollout-max-response-len 8192 --rollout-temperature 1.0 \
  --rm-type deepscaler --advantage-estimator grpo --eps-clip 0.2 --eps-clip-high 0.28 \
  --lr 1e-6 --weight-decay 0.1 --adam-beta1 0.9 --adam-beta2 0.98 --clip-grad 1.0 \
  --use-dynamic-batch-size --max-tokens-per-gpu 32768 --recompute-granularity full \
  --actor-num-nodes 1 --actor-num-gpus-per-node "$NGPU" --colocate \
  --expert-model-parallel-size "$NGPU" --use-rollout-routing-replay --sglang-mem-fraction-static 0.8 \
  --save-interval 20 --save "${SAVE_DIR:-/tmp/miles_b200_ckpt}"
