"""Tool calls in generated text: parsers for the markup of the common chat templates, execution through a user function,
and the observation messages that go back into the context.

``create_parser(name, tool_specs)`` returns ``parse(text) -> (plain text, [ToolCall])``. Names follow the function-call
parser names of the reference's engines (``--generate-tool-call-parser``):

* ``qwen25`` / ``qwen`` / ``hermes``:  ``<tool_call>{"name": ..., "arguments": {...}}</tool_call>``
* ``llama3``:  ``<|python_tag|>{"name": ..., "parameters": {...}}`` (several objects separated by ``;``), or a bare JSON
  object with those two keys
* ``mistral``:  ``[TOOL_CALLS] [{"name": ..., "arguments": {...}}, ...]``
* ``glm45`` / ``glm47``:  ``<tool_call>name\\n<arg_key>k</arg_key>\\n<arg_value>v</arg_value>...</tool_call>``
* ``deepseekv3``:  ``<｜tool▁call▁begin｜>function<｜tool▁sep｜>name\\n```json\\n{...}\\n```<｜tool▁call▁end｜>``

A call whose name is not among ``tool_specs`` (when given) is reported with ``name=None`` so that the environment can answer
with an error observation instead of raising. Values of the GLM form are JSON-decoded when they parse and kept as strings
otherwise.

Reference: miles/rollout/generate_utils/tool_call_utils.py:1-143 (which delegates the parsing to the engine package's
``FunctionCallParser``) and the execution loop of miles/rollout/generate_hub/multi_turn.py:26-98.
"""
from __future__ import annotations

import json
import re
import uuid
from dataclasses import dataclass, field
from typing import Any, Callable, Optional, Sequence


@dataclass
class ToolCall:
    name: Optional[str]
    arguments: dict = field(default_factory=dict)
    id: str = field(default_factory=lambda: f"call_{uuid.uuid4().hex[:24]}")
    error: Optional[str] = None


def _known(specs: Optional[Sequence[dict]]) -> Optional[set]:
    if not specs:
        return None
    names = set()
    for s in specs:
        fn = s.get("function", s) if isinstance(s, dict) else {}
        if fn.get("name"):
            names.add(fn["name"])
    return names or None


def _mk(obj: Any, known: Optional[set], args_key: Sequence[str] = ("arguments", "parameters")) -> ToolCall:
    if not isinstance(obj, dict) or not obj.get("name"):
        return ToolCall(None, {"raw": obj}, error="malformed tool call")
    args = next((obj[k] for k in args_key if k in obj), {})
    if isinstance(args, str):
        try:
            args = json.loads(args)
        except json.JSONDecodeError:
            return ToolCall(obj["name"], {"raw": args}, error="arguments are not JSON")
    if known is not None and obj["name"] not in known:
        return ToolCall(None, {"raw": obj}, error=f"unknown tool {obj['name']!r}")
    return ToolCall(obj["name"], args if isinstance(args, dict) else {"value": args})


def _json_or_error(text: str, known) -> list:
    try:
        obj = json.loads(text)
    except json.JSONDecodeError:
        return [ToolCall(None, {"raw": text}, error="malformed tool call")]
    return [_mk(o, known) for o in (obj if isinstance(obj, list) else [obj])]


_QWEN = re.compile(r"<tool_call>\s*(\{(?:(?!</?tool_call>).)*\})\s*</tool_call>", re.S)  # never across another call's tags
_GLM = re.compile(r"<tool_call>\s*([^\n<{]+?)\s*\n(.*?)</tool_call>", re.S)
_GLM_ARG = re.compile(r"<arg_key>(.*?)</arg_key>\s*<arg_value>(.*?)</arg_value>", re.S)
_DS = re.compile(r"<｜tool▁call▁begin｜>.*?<｜tool▁sep｜>\s*([^\n]+)\n```json\n(.*?)\n```\s*<｜tool▁call▁end｜>", re.S)


def _parse_qwen(text: str, known):
    calls = [c for m in _QWEN.finditer(text) for c in _json_or_error(m.group(1), known)]
    return _QWEN.sub("", text).strip(), calls


def _parse_llama3(text: str, known):
    if "<|python_tag|>" in text:
        head, tail = text.split("<|python_tag|>", 1)
        calls = [c for part in tail.split(";") if part.strip() for c in _json_or_error(part.strip().replace("<|eom_id|>", ""), known)]
        return head.strip(), calls
    s = text.strip()
    if s.startswith("{") and '"name"' in s:
        calls = _json_or_error(s, known)
        if all(c.error is None for c in calls):
            return "", calls
    return text, []


def _parse_mistral(text: str, known):
    if "[TOOL_CALLS]" not in text:
        return text, []
    head, tail = text.split("[TOOL_CALLS]", 1)
    return head.strip(), _json_or_error(tail.strip(), known)


def _parse_glm(text: str, known):
    calls = []
    for m in _GLM.finditer(text):
        name, body = m.group(1).strip(), m.group(2)
        args = {}
        for k, v in _GLM_ARG.findall(body):
            v = v.strip()
            try:
                args[k.strip()] = json.loads(v)
            except json.JSONDecodeError:
                args[k.strip()] = v
        calls.append(_mk({"name": name, "arguments": args}, known))
    return _GLM.sub("", text).strip(), calls


def _parse_deepseek(text: str, known):
    calls = []
    for m in _DS.finditer(text):
        try:
            calls.append(_mk({"name": m.group(1).strip(), "arguments": json.loads(m.group(2))}, known))
        except json.JSONDecodeError:
            calls.append(ToolCall(m.group(1).strip(), {"raw": m.group(2)}, error="arguments are not JSON"))
    plain = text.split("<｜tool▁calls▁begin｜>", 1)[0] if calls else text
    return plain.strip(), calls


PARSERS = {"qwen25": _parse_qwen, "qwen": _parse_qwen, "qwen3": _parse_qwen, "hermes": _parse_qwen, "llama3": _parse_llama3,
           "mistral": _parse_mistral, "glm45": _parse_glm, "glm47": _parse_glm, "glm": _parse_glm, "deepseekv3": _parse_deepseek}


def create_parser(name: Optional[str], tool_specs: Optional[Sequence[dict]] = None) -> Callable:
    fn = PARSERS.get((name or "qwen25").lower())
    if fn is None:
        raise ValueError(f"unknown tool-call parser {name!r}; known: {sorted(PARSERS)}")
    known = _known(tool_specs)
    return lambda text: fn(text or "", known)


async def execute_tool_calls(calls: Sequence[ToolCall], execute_one: Callable) -> list:
    """``execute_one(name, arguments) -> str`` (sync or async). One ``role: tool`` message per call; a failing or malformed
    call becomes an error observation (the model sees it and may try again), never an exception in the rollout."""
    out = []
    for c in calls:
        if c.error is not None or c.name is None:
            content = f"error: {c.error or 'malformed tool call'}"
        else:
            try:
                res = execute_one(c.name, c.arguments)
                if hasattr(res, "__await__"):
                    res = await res
                content = res if isinstance(res, str) else json.dumps(res)
            except Exception as e:  # noqa: BLE001
                content = f"error: {type(e).__name__}: {e}"
        out.append({"role": "tool", "tool_call_id": c.id, "name": c.name, "content": content})
    return out
