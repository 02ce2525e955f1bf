#!/usr/bin/env bash
# Two (or more) nodes: run this on every node with NODE_RANK = 0 .. NNODES-1 and MASTER_ADDR = the first node's address.
# Expert parallelism stays inside a node (8 GPUs, peer-memory kernels over NVLink), data parallelism spans the nodes: the
# groups that cross nodes use NCCL, the groups inside a node keep the fused kernels (miles_b200/parallel/topology.py decides
# per group). Every rank runs its own colocated rollout engine, so generation scales with the GPU count.
set -euo pipefail
NNODES=${NNODES:-2}
NODE_RANK=${NODE_RANK:-0}
MASTER_ADDR=${MASTER_ADDR:-127.0.0.1}
python -m torch.distributed.run --nnodes "$NNODES" --node-rank "$NODE_RANK" --nproc-per-node 8 \
  --master-addr "$MASTER_ADDR" --master-port 29500 train.py \
  --model-preset qwen3-30B-A3B ${HF_CHECKPOINT:+--hf-checkpoint "$HF_CHECKPOINT"} ${PROMPT_DATA:+--prompt-data "$PROMPT_DATA"} \
  --expert-model-parallel-size 8 --use-rollout-routing-replay \
  --num-rollout 100 --rollout-batch-size $((8 * 8 * NNODES)) --n-samples-per-prompt 8 --rollout-max-response-len 8192 \
  --rm-type deepscaler --advantage-estimator grpo --lr 1e-6 --use-dynamic-batch-size --max-tokens-per-gpu 32768 \
  --use-precision-aware-optimizer --exp-avg-dtype bf16 --exp-avg-sq-dtype bf16 --balance-data \
  --actor-num-nodes "$NNODES" --actor-num-gpus-per-node 8 --colocate \
  --save "${SAVE_DIR:-/tmp/miles_b200_ckpt}" --save-interval 20
