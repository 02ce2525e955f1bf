#!/usr/bin/env bash
# PPO with a critic of the same shape (chunked GAE, clipped value loss).
set -euo pipefail
NGPU=${NGPU:-4}
python -m torch.distributed.run --nnodes=1 --nproc-per-node "$NGPU" --master-addr 127.0.0.1 --master-port 29500 train.py \
  --model-preset qwen3-4B --advantage-estimator ppo --gamma 1.0 --lambd 0.95 --kl-coef 0.01 \
  --critic-lr 5e-6 --lr 1e-6 --num-rollout 100 --rollout-batch-size $((8 * NGPU)) --n-samples-per-prompt 1 \
  --rollout-max-response-len 4096 --rm-type deepscaler --use-dynamic-batch-size --max-tokens-per-gpu 16384 --colocate \
  --actor-num-nodes 1 --actor-num-gpus-per-node "$NGPU"
