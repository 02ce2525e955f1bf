#!/usr/bin/env bash
# GLM-4.5-Air (106B total, 12B active): sigmoid router with selection bias, one shared expert, rotary embedding on half of
# every head, a dense first layer. Expert parallel over all GPUs of the node; the HuggingFace checkpoint is read directly.
set -euo pipefail
NGPU=${NGPU:-8}
python -m torch.distributed.run --nnodes=1 --nproc-per-node "$NGPU" --master-addr 127.0.0.1 --master-port 29500 train.py \
  --model-preset glm4.5-106B-A12B ${HF_CHECKPOINT:+--hf-checkpoint "$HF_CHECKPOINT"} ${PROMPT_DATA:+--prompt-data "$PROMPT_DATA"} \
  --expert-model-parallel-size "$NGPU" --use-rollout-routing-replay --no-rollout-replicate-experts \
  --optimizer-cpu-offload --use-precision-aware-optimizer --exp-avg-dtype bf16 --exp-avg-sq-dtype bf16 \
  --num-rollout 100 --rollout-batch-size 32 --n-samples-per-prompt 8 --rollout-max-response-len 8192 \
  --rm-type deepscaler --advantage-estimator grpo --eps-clip 0.2 --eps-clip-high 0.28 --lr 1e-6 --weight-decay 0.1 \
  --use-dynamic-batch-size --max-tokens-per-gpu 16384 --recompute-granularity full \
  --actor-num-nodes 1 --actor-num-gpus-per-node "$NGPU" --colocate
