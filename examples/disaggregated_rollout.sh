#!/usr/bin/env bash
# Trainer and rollout engines on different GPUs of the box: engines are `miles_b200.engine.server` processes, the
# trainer generates over HTTP and pushes weights through a process group of its own (NCCL between the GPUs).
# GPUs 0..TRAIN-1 train (data parallel), GPUs TRAIN..7 serve. (`--launch-rollout-fleet --rollout-num-gpus N` makes the
# trainer start and stop the engine processes itself; this script starts them by hand to show the pieces.)
# With train_async.py the next rollout is generated while the current one trains.
set -euo pipefail
TRAIN=${TRAIN:-4}
MODEL=${MODEL:-qwen3-4B}
URLS=()
for ((g = TRAIN; g < 8; g++)); do
  port=$((30000 + g))
  CUDA_VISIBLE_DEVICES=$g python -m miles_b200.engine.server --model-preset "$MODEL" ${HF_CHECKPOINT:+--hf-checkpoint "$HF_CHECKPOINT"} \
    --port "$port" --max-running-requests 128 &
  URLS+=("http://127.0.0.1:$port")
done
trap 'kill $(jobs -p) 2>/dev/null || true' EXIT
IFS=, eval 'JOINED="${URLS[*]}"'
CUDA_VISIBLE_DEVICES=$(seq -s, 0 $((TRAIN - 1))) python -m torch.distributed.run --nnodes=1 --nproc-per-node "$TRAIN" \
  --master-addr 127.0.0.1 --master-port 29500 train_async.py \
  --model-preset "$MODEL" ${HF_CHECKPOINT:+--hf-checkpoint "$HF_CHECKPOINT"} ${PROMPT_DATA:+--prompt-data "$PROMPT_DATA"} \
  --rollout-engine-urls "$JOINED" --num-rollout 100 --rollout-batch-size 64 --n-samples-per-prompt 8 \
  --rollout-max-prompt-len 1024 --rollout-max-response-len 8192 --rm-type deepscaler --advantage-estimator grpo \
  --use-tis --lr 1e-6 --use-dynamic-batch-size --max-tokens-per-gpu 32768 --recompute-granularity full \
  --actor-num-nodes 1 --actor-num-gpus-per-node "$TRAIN"
