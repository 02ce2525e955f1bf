"""Hooks of the tree-serving session server: message matchers, the sample picker and the sample post-processor.

* a *message matcher* decides whether a message of a new request is "the same" as the one the session holds at that
  position, i.e. where a request stops extending a lineage and starts a branch (``--session-message-matcher``);
* the *picker* selects which of a session's leaf samples are trained (``--session-sample-picker-path``);
* the *post-processor* finalises them (``--session-sample-postprocessor-path``).

Reference: miles/rollout/session/v2/{matchers,picker_hub,postprocessor_hub}.py.
"""
from __future__ import annotations

import json
from typing import Callable


def _norm_tool_calls(calls) -> list:
    out = []
    for c in calls or []:
        fn = c.get("function", c)
        args = fn.get("arguments")
        if isinstance(args, str):
            try:
                args = json.loads(args)
            except ValueError:
                pass
        out.append((fn.get("name"), json.dumps(args, sort_keys=True, default=str)))
    return out


def match_strict(a: dict, b: dict) -> bool:
    """Role, content, tool calls (ids included) and tool-call id all equal."""
    keys = ("role", "content", "tool_calls", "tool_call_id", "name")
    return all((a.get(k) or None) == (b.get(k) or None) for k in keys)


def match_loose_tool_call(a: dict, b: dict) -> bool:
    """Like strict, but tool calls compare by function name and parsed arguments only: call ids and argument
    formatting may differ between what the policy emitted and what the agent framework echoes back."""
    if (a.get("role"), a.get("content") or None) != (b.get("role"), b.get("content") or None):
        return False
    return _norm_tool_calls(a.get("tool_calls")) == _norm_tool_calls(b.get("tool_calls"))


def match_role_content_only(a: dict, b: dict) -> bool:
    """Role and content only: different tool-call lineages with equal text collapse into one (an explicit opt-in)."""
    return (a.get("role"), a.get("content") or None) == (b.get("role"), b.get("content") or None)


MATCHERS = {"strict": match_strict, "loose_tool_call": match_loose_tool_call, "role_content_only": match_role_content_only}


def resolve_matcher(name: str) -> Callable[[dict, dict], bool]:
    if name in MATCHERS:
        return MATCHERS[name]
    from ...utils.misc import load_function

    return load_function(name.replace("miles.rollout.session.v2", "miles_b200.rollout.session"))


def drop_retries(leaf_samples: list, session_metadata: dict) -> list:
    """Default picker: when two leaves share their whole context and part ways at a *generated* token (the agent asked
    for the same turn again and got another answer), the earlier one is a superseded retry and is dropped; leaves that
    part ways inside context tokens (an edited or compacted history, a forked sub-agent) are separate lineages and
    are all kept."""
    def full_mask(s):
        return [0] * (len(s["tokens"]) - s["response_length"]) + list(s["loss_mask"])

    keep = []
    for i, s in enumerate(leaf_samples):
        ms = full_mask(s)
        superseded = False
        for t in leaf_samples[i + 1:]:
            mt = full_mask(t)
            n = min(len(s["tokens"]), len(t["tokens"]))
            k = 0
            while k < n and s["tokens"][k] == t["tokens"][k]:
                k += 1
            if k < n and ms[k] == 1 and mt[k] == 1:
                superseded = True
                break
        if not superseded:
            keep.append(s)
    return keep


def default_postprocess(leaf_samples: list, session_metadata: dict) -> list:
    """Default post-processor: a token that several kept leaves share (their common prefix) is trained exactly once,
    in the first leaf that contains it; rewards keyed by response id are attached when the session carries them."""
    seen: set = set()
    rewards = (session_metadata or {}).get("rewards", {})
    for s in leaf_samples:
        p = len(s["tokens"]) - s["response_length"]
        mask = list(s["loss_mask"])
        for k in range(len(mask)):
            key = (p + k, tuple(s["tokens"][:p + k + 1][-64:]), len(s["tokens"][:p + k + 1]))
            if mask[k] and key in seen:
                mask[k] = 0
            elif mask[k]:
                seen.add(key)
        s["loss_mask"] = mask
        rid = (s.get("metadata") or {}).get("response_id")
        if rid is not None and rid in rewards:
            s["reward"] = rewards[rid]
    return leaf_samples
