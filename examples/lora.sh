#!/usr/bin/env bash
# LoRA post-training: the base weights stay frozen (no optimizer state for them), only the adapters train; the colocated
# engine serves the merged weights, the adapter is saved in PEFT layout under <save>/iter_*/adapter.
# (Reference: examples/lora.)
set -euo pipefail
NGPU=${NGPU:-2}
python -m torch.distributed.run --nnodes=1 --nproc-per-node "$NGPU" --master-addr 127.0.0.1 --master-port 29500 train.py \
  --model-preset qwen3-4B ${HF_CHECKPOINT:+--hf-checkpoint "$HF_CHECKPOINT"} ${PROMPT_DATA:+--prompt-data "$PROMPT_DATA"} \
  --lora-rank 32 --lora-alpha 64 --target-modules all-linear ${LORA_ADAPTER:+--lora-adapter-path "$LORA_ADAPTER"} \
  --num-rollout 100 --rollout-batch-size $((8 * NGPU)) --n-samples-per-prompt 8 --rollout-max-response-len 4096 \
  --rm-type deepscaler --advantage-estimator grpo --lr 1e-5 --use-dynamic-batch-size --max-tokens-per-gpu 32768 \
  --actor-num-nodes 1 --actor-num-gpus-per-node "$NGPU" --colocate --check-lora-weight-equal \
  --save "${SAVE_DIR:-/tmp/miles_b200_lora}" --save-interval 20
