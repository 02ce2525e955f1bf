"""Multi-turn generation with tool calls.

Each turn generates until a stop; tool calls found in the text are executed through the user's tool
module (``--custom-tool-path`` style object with ``async call(name, args)``) and the tool output is
appended to the context as observation tokens with loss-mask 0, so that only model-written tokens are
trained on (reference: miles/rollout/generate_hub/multi_turn.py:26-98).  The loop ends on a final
answer, on ``max_turns`` or when the context budget is exhausted.
"""
from __future__ import annotations

import json
import re
from typing import Any

from ...utils.misc import load_function
from ...utils.types import Sample
from ..base_types import GenerateFnInput, GenerateFnOutput
from .common import compute_request_payload, prompt_ids, update_sample_from_response

_TOOL_RE = re.compile(r"<tool_call>\s*(\{.*?\})\s*</tool_call>", re.S)


def add_arguments(parser) -> None:
    parser.add_argument("--generate-max-turns", type=int, default=8)
    parser.add_argument("--generate-tool-module-path", type=str, default=None)
    # the reference's names: a function ``execute(name, arguments) -> str``, the tool specifications shown to the model,
    # and the markup its calls are written in (rollout/generate_hub/tool_calls.py)
    parser.add_argument("--generate-execute-tool-function-path", type=str, default=None)
    parser.add_argument("--generate-tool-specs-path", type=str, default=None)
    parser.add_argument("--generate-tool-call-parser", type=str, default=None)
    parser.add_argument("--generate-observation-template", type=str, default="\n<tool_response>\n{result}\n</tool_response>\n")


def parse_tool_calls(text: str) -> list:
    calls = []
    for m in _TOOL_RE.finditer(text or ""):
        try:
            obj = json.loads(m.group(1))
            calls.append((obj.get("name"), obj.get("arguments", {})))
        except json.JSONDecodeError:
            calls.append((None, {"raw": m.group(1)}))
    return calls


async def _run_tools(tool_module: Any, calls: list) -> str:
    outs = []
    for name, arguments in calls:
        if name is None:
            outs.append("error: malformed tool call")
            continue
        try:
            res = tool_module.call(name, arguments)
            if hasattr(res, "__await__"):
                res = await res
            outs.append(res if isinstance(res, str) else json.dumps(res))
        except Exception as e:  # noqa: BLE001 - a failing tool is an observation, not a crash
            outs.append(f"error: {type(e).__name__}: {e}")
    return "\n".join(outs)


async def generate(inp: GenerateFnInput) -> GenerateFnOutput:
    state, sample = inp.state, inp.sample
    a = state.args
    assert state.tokenizer is not None, "multi-turn generation needs a tokenizer"
    tool_module = load_function(a.generate_tool_module_path) if getattr(a, "generate_tool_module_path", None) else None
    execute_one = load_function(a.generate_execute_tool_function_path) if getattr(a, "generate_execute_tool_function_path", None) else None
    parser = None
    if execute_one is not None or getattr(a, "generate_tool_call_parser", None):
        from .tool_calls import create_parser

        specs = load_function(a.generate_tool_specs_path) if getattr(a, "generate_tool_specs_path", None) else None
        parser = create_parser(getattr(a, "generate_tool_call_parser", None), specs() if callable(specs) else specs)
    max_turns = getattr(a, "generate_max_turns", 8)
    template = getattr(a, "generate_observation_template", "\n<tool_response>\n{result}\n</tool_response>\n")
    budget = inp.sampling_params["max_new_tokens"]
    ids = prompt_ids(state, sample)
    sample.tokens, sample.loss_mask, sample.response_length = list(ids), [], 0
    sample.rollout_log_probs = []
    for turn in range(max_turns):
        sp = dict(inp.sampling_params)
        sp["max_new_tokens"] = budget - sample.response_length
        payload = compute_request_payload(state, sample, list(sample.tokens), sp)
        if payload is None:
            sample.status = Sample.Status.TRUNCATED
            break
        out = await state.client.generate(payload)
        before = sample.response_length
        update_sample_from_response(state, sample, sample.tokens, out, loss_mask_value=1)
        sample.loss_mask = sample.loss_mask[:before] + [1] * (sample.response_length - before)
        sample.metadata["turns"] = turn + 1
        if sample.status != Sample.Status.COMPLETED:
            break
        if parser is not None:
            from .tool_calls import execute_tool_calls

            _, found = parser(out.get("text", ""))
            if not found or (execute_one is None and tool_module is None):
                break
            run = execute_one if execute_one is not None else tool_module.call
            msgs = await execute_tool_calls(found, run)
            obs = template.format(result="\n".join(m["content"] for m in msgs))
        else:
            calls = parse_tool_calls(out.get("text", ""))
            if not calls or tool_module is None:
                break
            obs = template.format(result=await _run_tools(tool_module, calls))
        obs_ids = state.tokenizer(obs, add_special_tokens=False)["input_ids"]
        if sample.response_length + len(obs_ids) >= budget:
            sample.status = Sample.Status.TRUNCATED
            break
        sample.tokens += obs_ids
        sample.response += obs
        sample.response_length += len(obs_ids)
        sample.loss_mask += [0] * len(obs_ids)
        sample.rollout_log_probs += [0.0] * len(obs_ids)
    return GenerateFnOutput(samples=sample)


generate.add_arguments = add_arguments
