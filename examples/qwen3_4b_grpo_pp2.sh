#!/usr/bin/env bash
# Qwen3-4B GRPO, pipeline parallel 2 x data parallel NGPU/2: every stage keeps half of the layers, the colocated
# engines decode on a full-model replica that the weight update fills stage by stage, all GPUs generate.
set -euo pipefail
NGPU=${NGPU:-8}
python -m torch.distributed.run --nnodes=1 --nproc-per-node "$NGPU" --master-addr 127.0.0.1 --master-port 29500 train.py \
  --model-preset qwen3-4B ${HF_CHECKPOINT:+--hf-checkpoint "$HF_CHECKPOINT"} ${PROMPT_DATA:+--prompt-data "$PROMPT_DATA"} \
  --pipeline-model-parallel-size 2 --num-rollout 100 --rollout-batch-size $((8 * NGPU)) --n-samples-per-prompt 8 \
  --rollout-max-prompt-len 1024 --rollout-max-response-len 8192 --rollout-temperature 1.0 \
  --rm-type deepscaler --advantage-estimator grpo --eps-clip 0.2 --eps-clip-high 0.28 \
  --lr 1e-6 --weight-decay 0.1 --clip-grad 1.0 --use-dynamic-batch-size --max-tokens-per-gpu 16384 \
  --recompute-granularity full --actor-num-nodes 1 --actor-num-gpus-per-node "$NGPU" --colocate
