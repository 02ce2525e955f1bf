#!/usr/bin/env bash
# Multi-turn agent rollouts: `my_agent.agent(chat, sample, args)` is a coroutine that talks to the policy through an
# OpenAI-style `chat(messages)`; the session keeps the exact tokens, tool / user turns are masked out of the loss.
#
#   async def agent(chat, sample, args):
#       msgs = [{"role": "user", "content": sample.prompt}]
#       for _ in range(4):
#           a = await chat(msgs)
#           msgs.append({"role": "assistant", "content": a["content"]})
#           tool = run_tool(a["content"])
#           if tool is None: break
#           msgs.append({"role": "tool", "content": tool})
#       return {"final": msgs[-1]["content"]}
set -euo pipefail
NGPU=${NGPU:-8}
python -m torch.distributed.run --nnodes=1 --nproc-per-node "$NGPU" --master-addr 127.0.0.1 --master-port 29500 train.py \
  --model-preset qwen3-4B --hf-checkpoint "$HF_CHECKPOINT" --prompt-data "$PROMPT_DATA" --input-key prompt --label-key label \
  --custom-generate-function-path miles_b200.rollout.generate_hub.agentic.generate \
  --custom-agent-function-path "${AGENT:-my_agent.agent}" --tito-family qwen3 \
  --num-rollout 100 --rollout-batch-size $((4 * NGPU)) --n-samples-per-prompt 8 \
  --rollout-max-response-len 8192 --rm-type "${RM_TYPE:-f1}" --advantage-estimator grpo \
  --lr 1e-6 --use-dynamic-batch-size --max-tokens-per-gpu 32768 --recompute-granularity full \
  --actor-num-nodes 1 --actor-num-gpus-per-node "$NGPU" --colocate
