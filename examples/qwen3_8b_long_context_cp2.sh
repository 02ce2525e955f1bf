#!/usr/bin/env bash
# Qwen3-8B GRPO with long responses: context parallel 2 x data parallel NGPU/2. On the sm_100a path every rank holds a
# shard of each sequence and trades it for a head shard around the attention kernels (all-to-all over NVSwitch), so a
# 64K-token sample needs a 32K-token activation footprint per GPU. (Reference: --context-parallel-size in
# scripts/run_qwen3_4B.py and docs/advanced/long-context.)
set -euo pipefail
NGPU=${NGPU:-8}
python -m torch.distributed.run --nnodes=1 --nproc-per-node "$NGPU" --master-addr 127.0.0.1 --master-port 29500 train.py \
  --model-preset qwen3-8B ${HF_CHECKPOINT:+--hf-checkpoint "$HF_CHECKPOINT"} ${PROMPT_DATA:+--prompt-data "$PROMPT_DATA"} \
  --context-parallel-size 2 --num-rollout 100 --rollout-batch-size $((4 * NGPU / 2)) --n-samples-per-prompt 8 \
  --rollout-max-prompt-len 2048 --rollout-max-response-len 61440 --rollout-temperature 1.0 \
  --rm-type deepscaler --advantage-estimator grpo --eps-clip 0.2 --eps-clip-high 0.28 \
  --lr 1e-6 --weight-decay 0.1 --clip-grad 1.0 --use-dynamic-batch-size --max-tokens-per-gpu 65536 \
  --actor-num-nodes 1 --actor-num-gpus-per-node "$NGPU" --colocate
