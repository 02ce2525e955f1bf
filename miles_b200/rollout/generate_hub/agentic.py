"""Agentic generation: a user-written agent talks to the policy through an OpenAI-style chat interface, the session
behind it records the exact tokens, and the finished session becomes the training sample.

The agent is a coroutine ``agent(chat, sample, args) -> Optional[dict]`` found at ``--custom-agent-function-path``;
``chat(messages, **sampling)`` returns the assistant message (``{"role": "assistant", "content": ...}``) and keeps
the conversation's token sequence in a token-in-token-out session (`rollout/session/`): generated tokens are trained
on, everything the environment contributed (system / user / tool messages) is masked out. Whatever the agent
returns is stored in ``sample.metadata["agent_result"]`` for the reward function. The same agent code can run against
the HTTP session server (``/sessions/{id}/v1/chat/completions``) outside the trainer.

Reference counterpart: miles/rollout/generate_hub/agentic_tool_call.py (OpenAI-endpoint agent through the session server).
"""
from __future__ import annotations

import asyncio
import uuid
from typing import Any

from ...utils.misc import load_function
from ...utils.types import Sample
from ..base_types import GenerateFnInput, GenerateFnOutput
from ..session.tito import TitoTokenizer
from ..session.trajectory import LinearTrajectory


class SessionChat:
    """The ``chat`` callable handed to the agent: one linear token-in-token-out session over the engine client."""

    def __init__(self, state, sampling_params: dict, routing_key: str):
        self.state, self.sp, self.routing_key = state, dict(sampling_params), routing_key
        self.tito = TitoTokenizer(state.tokenizer, getattr(state.args, "tito_family", None))
        self.traj = LinearTrajectory(routing_key)
        self.num_messages = 0
        self.routed = None
        self.budget = self.sp.get("max_new_tokens", 1 << 30)   # response tokens the whole session may produce

    async def __call__(self, messages: list, **overrides: Any) -> dict:
        if len(messages) < self.num_messages:
            raise ValueError("a session only moves forward: the request holds fewer messages than the session")
        if not self.traj.tokens:
            self.traj.append_context(messages[-1]["role"] if messages else "user", self.tito.initial(messages, overrides.pop("tools", None)))
        else:
            new = [m for m in messages[self.num_messages:] if m.get("role") != "assistant"]
            last = self.traj.turns[-1]
            self.traj.append_context(new[-1]["role"] if new else "user",
                                     self.tito.continuation(self.traj.tokens[last.start:last.end], new))
        used = len(self.traj.tokens) - self.traj.prompt_length
        sp = dict(self.sp)
        sp.update({k: v for k, v in overrides.items() if k in ("temperature", "top_p", "top_k", "stop", "stop_token_ids")})
        sp["max_new_tokens"] = min(int(overrides.get("max_tokens", sp.get("max_new_tokens", 1024))), max(self.budget - used, 0))
        if sp["max_new_tokens"] <= 0:
            self.traj.finish_reason = "length"
            return {"role": "assistant", "content": "", "finish_reason": "length"}
        payload = {"input_ids": list(self.traj.tokens), "sampling_params": sp, "return_logprob": True, "routing_key": self.routing_key}
        if getattr(self.state.args, "use_rollout_routing_replay", False):
            payload["return_routed_experts"] = True
        out = await self.state.client.generate(payload)
        meta = out["meta_info"]
        ids = list(out["output_ids"])
        self.traj.append_generation(ids, [lp for lp, _ in meta.get("output_token_logprobs", [])] or [0.0] * len(ids),
                                    meta.get("weight_version"), meta["finish_reason"]["type"])
        from ...engine.client import decode_routed_experts

        re = decode_routed_experts(meta)
        if re is not None:
            self.routed = re  # routing of the whole context so far (the last request covers every earlier token)
        self.num_messages = len(messages) + 1
        text = out.get("text")
        if text is None and hasattr(self.state.tokenizer, "decode"):
            text = self.state.tokenizer.decode(ids, skip_special_tokens=True)
        return {"role": "assistant", "content": text or "", "finish_reason": meta["finish_reason"]["type"]}


async def generate(inp: GenerateFnInput) -> GenerateFnOutput:
    state, sample = inp.state, inp.sample
    path = getattr(state.args, "custom_agent_function_path", None)
    if not path:
        raise ValueError("agentic generation needs --custom-agent-function-path")
    agent = load_function(path)
    chat = SessionChat(state, inp.sampling_params, sample.routing_key or uuid.uuid4().hex)
    result = agent(chat, sample, state.args)
    if asyncio.iscoroutine(result):
        result = await result
    d = chat.traj.to_sample_dict()
    sample.tokens = d["tokens"]
    sample.response_length = d["response_length"]
    sample.loss_mask = d["loss_mask"]
    sample.rollout_log_probs = d["rollout_log_probs"]
    sample.weight_versions = d["weight_versions"]
    if chat.routed is not None:
        sample.rollout_routed_experts = chat.routed
    if hasattr(state.tokenizer, "decode"):
        p = len(d["tokens"]) - d["response_length"]
        sample.response = state.tokenizer.decode(d["tokens"][p:], skip_special_tokens=False)
    sample.metadata = dict(sample.metadata or {}, agent_result=result, turns=d["metadata"]["turns"])
    sample.status = Sample.Status.TRUNCATED if d["status"] == "truncated" else Sample.Status.COMPLETED
    if d["response_length"] == 0:
        sample.status = Sample.Status.FAILED
    return GenerateFnOutput(samples=sample)
