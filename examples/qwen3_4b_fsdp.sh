#!/usr/bin/env bash
# Sharded data parallelism (the reference's FSDP backend): every GPU keeps 1/N of each decoder layer's parameters, fp32
# master weights and Adam moments; layers are all-gathered (with prefetch) for compute and their gradients reduce-scattered
# in the backward. --dp-replicate-size 2 would run two replicas of a model sharded over N/2 GPUs each. The flags may also
# come from a YAML file: --config fsdp.yaml (keys are flag names with underscores; unknown keys are an error).
set -euo pipefail
NGPU=${NGPU:-8}
python -m torch.distributed.run --nnodes=1 --nproc-per-node "$NGPU" --master-addr 127.0.0.1 --master-port 29500 train.py \
  --train-backend fsdp --dp-replicate-size "${REPLICAS:-1}" \
  --model-preset qwen3-4B ${HF_CHECKPOINT:+--hf-checkpoint "$HF_CHECKPOINT"} ${PROMPT_DATA:+--prompt-data "$PROMPT_DATA"} \
  --num-rollout 100 --rollout-batch-size $((8 * NGPU)) --n-samples-per-prompt 8 --rollout-max-response-len 4096 \
  --rm-type deepscaler --advantage-estimator grpo --lr 1e-6 --use-dynamic-batch-size --max-tokens-per-gpu 32768 \
  --actor-num-nodes 1 --actor-num-gpus-per-node "$NGPU" --colocate --save "${SAVE_DIR:-/tmp/miles_b200_fsdp}" --save-interval 20
