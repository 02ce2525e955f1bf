#!/usr/bin/env bash
# On-policy distillation: the student's samples are scored by teacher servers during the rollout and every sampled token is
# penalised by opd_kl_coef * (student log-prob - teacher log-prob). Teachers are engine servers of this package (any server
# that answers /generate with max_new_tokens = 0 and return_logprob works); samples choose their teacher through
# metadata["opd_teacher"], others go to the entry called "default". (Reference: examples/on_policy_distillation.)
set -euo pipefail
NGPU=${NGPU:-4}
# teachers on the last two GPUs:
#   CUDA_VISIBLE_DEVICES=6 python -m miles_b200.engine.server --hf-checkpoint "$TEACHER_A" --port 31000 &
#   CUDA_VISIBLE_DEVICES=7 python -m miles_b200.engine.server --hf-checkpoint "$TEACHER_B" --port 31001 &
python -m torch.distributed.run --nnodes=1 --nproc-per-node "$NGPU" --master-addr 127.0.0.1 --master-port 29500 train.py \
  --model-preset qwen3-4B ${HF_CHECKPOINT:+--hf-checkpoint "$HF_CHECKPOINT"} ${PROMPT_DATA:+--prompt-data "$PROMPT_DATA"} \
  --use-opd --opd-type sglang --opd-kl-coef 1.0 \
  --opd-teacher-urls default=http://127.0.0.1:31000/generate math=http://127.0.0.1:31001/generate --opd-teacher-key opd_teacher \
  --num-rollout 100 --rollout-batch-size $((8 * NGPU)) --n-samples-per-prompt 4 --rollout-max-response-len 4096 \
  --advantage-estimator grpo --lr 1e-6 --use-dynamic-batch-size --max-tokens-per-gpu 32768 \
  --actor-num-nodes 1 --actor-num-gpus-per-node "$NGPU" --colocate
