#!/usr/bin/env bash
# Fully asynchronous rollout: generation keeps running while the trainer steps; samples older than
# --max-weight-staleness weight versions are dropped (reference: examples/fully_async).
set -euo pipefail
NGPU=${NGPU:-8}
python -m torch.distributed.run --nnodes=1 --nproc-per-node "$NGPU" --master-addr 127.0.0.1 --master-port 29500 train_async.py \
  --model-preset qwen3-30B-A3B --fully-async --max-weight-staleness 2 --update-weights-interval 1 \
  --num-rollout 100 --rollout-batch-size $((8 * NGPU)) --n-samples-per-prompt 8 --rollout-max-response-len 8192 \
  --rm-type deepscaler --advantage-estimator grpo --use-tis --lr 1e-6 --use-dynamic-batch-size --max-tokens-per-gpu 32768 \
  --expert-model-parallel-size "$NGPU" --use-rollout-routing-replay --actor-num-nodes 1 --actor-num-gpus-per-node "$NGPU"
