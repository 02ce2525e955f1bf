#!/usr/bin/env bash
# Importance-sampling correction of the trainer / rollout-engine mismatch with variance controls (levels, bounds,
# rejection sampling, veto): the plug-in miles_b200.rl.mis.mis_function with the options of mis.yaml next to this file.
# --get-mismatch-metrics alone (without --use-tis) only reports the mismatch metrics.
set -euo pipefail
HERE="$(cd "$(dirname "$0")" && pwd)"
NGPU=${NGPU:-4}
python -m torch.distributed.run --nnodes=1 --nproc-per-node "$NGPU" --master-addr 127.0.0.1 --master-port 29500 "$HERE/../../train.py" \
  --model-preset qwen3-4B ${HF_CHECKPOINT:+--hf-checkpoint "$HF_CHECKPOINT"} ${PROMPT_DATA:+--prompt-data "$PROMPT_DATA"} \
  --use-tis --get-mismatch-metrics --custom-tis-function-path miles_b200.rl.mis.mis_function \
  --custom-config-path "$HERE/mis.yaml" \
  --num-rollout 100 --rollout-batch-size $((8 * NGPU)) --n-samples-per-prompt 8 --rollout-max-response-len 4096 \
  --rm-type deepscaler --advantage-estimator grpo --lr 1e-6 --use-dynamic-batch-size --max-tokens-per-gpu 32768 \
  --actor-num-nodes 1 --actor-num-gpus-per-node "$NGPU" --colocate
