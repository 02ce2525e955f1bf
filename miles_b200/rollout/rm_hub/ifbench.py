"""A small instruction-following checker: verifies the verifiable constraints listed in the label.

``label`` (or ``metadata['instructions']``) is a list of dicts such as ``{"type": "max_words", "value": 50}``,
``{"type": "contains", "value": "foo"}``, ``{"type": "num_paragraphs", "value": 3}``, ``{"type": "all_lowercase"}``,
``{"type": "ends_with", "value": "..."}``; the score is the fraction of satisfied constraints.
"""
from __future__ import annotations

import json
import re


def _check(resp: str, ins: dict) -> bool:
    t, v = ins.get("type"), ins.get("value")
    words = resp.split()
    if t == "max_words":
        return len(words) <= int(v)
    if t == "min_words":
        return len(words) >= int(v)
    if t == "contains":
        return str(v).lower() in resp.lower()
    if t == "not_contains":
        return str(v).lower() not in resp.lower()
    if t == "num_paragraphs":
        return len([p for p in re.split(r"\n\s*\n", resp.strip()) if p.strip()]) == int(v)
    if t == "all_lowercase":
        return resp == resp.lower()
    if t == "all_uppercase":
        return resp == resp.upper()
    if t == "ends_with":
        return resp.strip().endswith(str(v))
    if t == "starts_with":
        return resp.strip().startswith(str(v))
    if t == "json":
        try:
            json.loads(resp)
            return True
        except Exception:
            return False
    if t == "num_bullets":
        return len(re.findall(r"^\s*[-*] ", resp, flags=re.M)) == int(v)
    return False


def score_instruction_following(response: str, label, metadata=None) -> float:
    ins = label if isinstance(label, list) else (metadata or {}).get("instructions")
    if isinstance(label, str):
        try:
            ins = json.loads(label)
        except Exception:
            ins = ins or []
    if not ins:
        return 0.0
    return sum(_check(response or "", i) for i in ins) / len(ins)
