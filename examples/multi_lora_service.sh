#!/usr/bin/env bash
# Several LoRA adapters on one base model; adapters are added and removed over HTTP while the service runs:
#   curl -X POST localhost:8068/adapters -d '{"name": "math-a", "rank": 16, "lr": 1e-4}'
#   curl -X POST localhost:8068/adapters -d '{"name": "code-c", "rank": 8, "prompt_data": "/data/code.jsonl", "input_key": "prompt",
#        "label_key": "tests", "rm_type": "remote_rm", "rollout_batch_size": 4, "num_epoch": 2}'   # own data, reward, batch, lifetime
#   curl localhost:8068/adapters
#   curl -X DELETE localhost:8068/adapters/math-a
# An adapter with num_step / num_epoch retires by itself: it is saved under $SAVE_DIR/<name>/final_step_N and its slot is freed.
set -euo pipefail
NGPU=${NGPU:-1}
python -m torch.distributed.run --nnodes=1 --nproc-per-node "$NGPU" --master-addr 127.0.0.1 --master-port 29500 train_multi_lora_async.py \
  --model-preset qwen3-4B --lora-rank 16 --lora-alpha 32 --multi-lora-n-adapters 8 --multi-lora-api-port 8068 \
  --multi-lora-adapter math-a none --multi-lora-adapter code-b none \
  --rollout-batch-size 8 --n-samples-per-prompt 8 --rollout-max-response-len 2048 --rm-type deepscaler \
  --advantage-estimator grpo --lr 1e-4 --colocate --save "${SAVE_DIR:-/tmp/miles_b200_adapters}" --save-interval 10
