"""Reward hub: ``async_rm(args, sample)`` / ``batched_async_rm(args, samples)`` dispatch on ``--rm-type``.

Built-in types follow the reference's miles/rollout/rm_hub/__init__.py:19-109: ``remote_rm`` (HTTP POST to
``--rm-url``), ``deepscaler``, ``dapo``, ``math``, ``f1``, ``gpqa``, ``ifbench``, ``random``,
``deterministic_random``; a ``boxed_`` prefix extracts the last ``\\boxed{}`` answer first;
``--custom-rm-path`` replaces the dispatcher; ``--group-rm`` scores whole groups at once.  ``parity`` is
the synthetic reward of the benchmark configurations (1.0 when the response token-id sum is even).
"""
from __future__ import annotations

import asyncio
import hashlib
import random
from typing import Optional, Sequence

from ...utils.misc import load_function
from ...utils.types import Sample
from .math_utils import extract_boxed, grade_math_answer, normalize_answer
from .f1 import f1_score


def _response_tokens(sample: Sample) -> list:
    return list(sample.tokens[len(sample.tokens) - sample.response_length:]) if sample.response_length else []


async def remote_rm(args, sample: Sample) -> float:
    import aiohttp

    payload = {"prompt": sample.prompt, "response": sample.response, "label": sample.label}
    async with aiohttp.ClientSession() as sess:
        async with sess.post(args.rm_url, json=payload) as resp:
            resp.raise_for_status()
            return await resp.json()


def _rm_sync(rm_type: str, sample: Sample, args=None):
    response, label = sample.response, sample.label
    if rm_type.startswith("boxed_"):
        response = extract_boxed(response) or ""
        rm_type = rm_type[len("boxed_"):]
    if rm_type == "parity":
        return 1.0 if sum(_response_tokens(sample)) % 2 == 0 else 0.0
    if rm_type in ("deepscaler", "math", "dapo", "gemma_math"):
        ans = response
        if rm_type in ("deepscaler", "gemma_math") and "</think>" in response:
            ans = response.split("</think>")[-1]
        ok = grade_math_answer(ans, str(label) if label is not None else "")
        if rm_type == "dapo":
            return 1.0 if ok else -1.0
        return 1.0 if ok else 0.0
    if rm_type == "f1":
        return f1_score(response, str(label))[0]
    if rm_type == "gpqa":
        pred = normalize_answer(extract_boxed(response) or response.strip()[-1:] or "")
        return 1.0 if pred.upper() == str(label).strip().upper() else 0.0
    if rm_type == "ifbench":
        from .ifbench import score_instruction_following

        return score_instruction_following(response, label, sample.metadata)
    if rm_type == "random":
        return float(random.randint(0, 1))
    if rm_type == "deterministic_random":
        h = hashlib.sha256((str(sample.prompt) + "|" + sample.response).encode()).digest()
        return float(h[0] & 1)
    raise NotImplementedError(f"rm_type {rm_type!r} is not implemented")


async def async_rm(args, sample: Sample, **kwargs):
    if getattr(args, "custom_rm_path", None):
        fn = load_function(args.custom_rm_path)
        out = fn(args, sample, **kwargs)
        return await out if asyncio.iscoroutine(out) else out
    spec = getattr(sample, "reward_spec", None)
    rm_type = (spec.get("rm_type") if isinstance(spec, dict) else None) or (sample.metadata or {}).get("rm_type") or args.rm_type
    if rm_type is None:
        raise ValueError("no --rm-type / --custom-rm-path configured")
    if rm_type == "remote_rm":
        return await remote_rm(args, sample)
    return _rm_sync(rm_type.strip(), sample, args)


async def batched_async_rm(args, samples: Sequence[Sample], **kwargs) -> list:
    if getattr(args, "custom_rm_path", None) and getattr(args, "group_rm", False):
        fn = load_function(args.custom_rm_path)
        out = fn(args, list(samples), **kwargs)
        return await out if asyncio.iscoroutine(out) else out
    return list(await asyncio.gather(*[async_rm(args, s, **kwargs) for s in samples]))
