#!/usr/bin/env bash
# Qwen3-30B-A3B GRPO with a block-scaled rollout engine: training stays bf16, the engine multiplies MXFP8 (or NVFP4)
# copies of the projections and experts that every weight update re-quantises; importance-sampling correction (TIS)
# absorbs the train / rollout mismatch the lower precision adds.
set -euo pipefail
NGPU=${NGPU:-8}
QUANT=${QUANT:-mxfp8}
python -m torch.distributed.run --nnodes=1 --nproc-per-node "$NGPU" --master-addr 127.0.0.1 --master-port 29500 train.py \
  --model-preset qwen3-30B-A3B ${HF_CHECKPOINT:+--hf-checkpoint "$HF_CHECKPOINT"} ${PROMPT_DATA:+--prompt-data "$PROMPT_DATA"} \
  --expert-model-parallel-size "$NGPU" --rollout-quantization "$QUANT" --use-tis --use-rollout-routing-replay \
  --num-rollout 100 --rollout-batch-size $((8 * NGPU)) --n-samples-per-prompt 8 \
  --rollout-max-prompt-len 1024 --rollout-max-response-len 8192 --rollout-temperature 1.0 \
  --rm-type deepscaler --advantage-estimator grpo --eps-clip 0.2 --eps-clip-high 0.28 \
  --lr 1e-6 --weight-decay 0.1 --clip-grad 1.0 --use-dynamic-batch-size --max-tokens-per-gpu 32768 \
  --recompute-granularity full --actor-num-nodes 1 --actor-num-gpus-per-node "$NGPU" --colocate
