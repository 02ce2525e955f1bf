"""Look at, re-score and re-send what ``--save-debug-rollout-data`` wrote.

    python -m miles_b200.tools.debug_rollout_data show  rollout_3.pt [--limit 8] [--tokenizer DIR]
    python -m miles_b200.tools.debug_rollout_data score rollout_3.pt --rm-type deepscaler | --custom-rm-path pkg.mod.fn
    python -m miles_b200.tools.debug_rollout_data send  rollout_3.pt --url http://127.0.0.1:30000 [--limit 4] [--max-new-tokens 64]

``show``  prints one block per sample (index, status, reward, lengths, head of prompt and response) and the summary a
          training step would log (reward mean, length percentiles, truncated share).
``score`` runs a reward function over the saved samples again and reports where the new reward differs from the saved one
          (a changed grader, a flaky remote judge).
``send``  posts the saved prompts to an engine's ``/generate`` and prints what comes back now.

Reference: miles/utils/debug_utils/{display_debug_rollout_data,replay_reward_fn,send_to_sglang}.py.
"""
from __future__ import annotations

import argparse
import asyncio
import sys
from typing import Optional

import torch

from ..utils.types import Sample


def load_samples(path: str) -> list:
    pack = torch.load(path, map_location="cpu", weights_only=False)
    return [Sample.from_dict(d) for d in pack["samples"]]


def _short(text, n: int = 160) -> str:
    if text is None:
        return ""
    s = str(text).replace("\n", "\\n")
    return s if len(s) <= n else s[:n] + "..."


def _reward(s: Sample) -> Optional[float]:
    r = s.reward
    if isinstance(r, dict):
        r = next((v for v in r.values() if isinstance(v, (int, float))), None)
    return float(r) if isinstance(r, (int, float)) else None


def summarize(samples: list) -> dict:
    rewards = [r for r in (_reward(s) for s in samples) if r is not None]
    lens = sorted(int(s.response_length or 0) for s in samples)
    pick = lambda q: lens[min(len(lens) - 1, int(q * len(lens)))] if lens else 0  # noqa: E731
    status = [getattr(s.status, "value", s.status) for s in samples]
    return {"samples": len(samples), "reward_mean": sum(rewards) / len(rewards) if rewards else None,
            "reward_nonzero_frac": sum(1 for r in rewards if r != 0) / len(rewards) if rewards else None,
            "response_len_p50": pick(0.5), "response_len_p90": pick(0.9), "response_len_max": lens[-1] if lens else 0,
            "truncated_frac": sum(1 for x in status if str(x).lower().endswith("truncated")) / max(len(status), 1)}


def show(samples: list, limit: int = 8, tokenizer=None, out=sys.stdout) -> dict:
    for i, s in enumerate(samples[:limit]):
        prompt, resp = s.prompt, s.response
        if tokenizer is not None and s.tokens:
            n = int(s.response_length or 0)
            prompt = tokenizer.decode(s.tokens[:len(s.tokens) - n])
            resp = tokenizer.decode(s.tokens[len(s.tokens) - n:])
        print(f"--- sample {i + 1}/{len(samples)}  index={s.index} status={getattr(s.status, 'value', s.status)} reward={s.reward} "
              f"tokens={len(s.tokens or [])} response_length={s.response_length}", file=out)
        print(f"    prompt:   {_short(prompt)}", file=out)
        print(f"    response: {_short(resp)}", file=out)
    summary = summarize(samples)
    print("--- " + " ".join(f"{k}={v:.4g}" if isinstance(v, float) else f"{k}={v}" for k, v in summary.items()), file=out)
    return summary


async def rescore(samples: list, rm_type: Optional[str] = None, custom_rm_path: Optional[str] = None, out=sys.stdout) -> list:
    """Returns ``[(index, saved reward, new reward)]`` for the samples whose reward changed."""
    from types import SimpleNamespace

    from ..rollout.rm_hub import async_rm

    args = SimpleNamespace(rm_type=rm_type, custom_rm_path=custom_rm_path, group_rm=False)
    new = await asyncio.gather(*[async_rm(args, s) for s in samples])
    changed = []
    for s, r in zip(samples, new):
        old = _reward(s)
        r_num = r if isinstance(r, (int, float)) else _reward(SimpleNamespace(reward=r))
        if old is None or r_num is None or abs(float(old) - float(r_num)) > 1e-9:
            changed.append((s.index, s.reward, r))
    print(f"{len(changed)} of {len(samples)} rewards differ from the saved ones", file=out)
    for idx, old, r in changed[:20]:
        print(f"    index={idx} saved={old} now={r}", file=out)
    return changed


async def send(samples: list, url: str, limit: int = 4, max_new_tokens: int = 64, temperature: float = 0.0, out=sys.stdout, post=None) -> list:
    from ..utils import http_utils

    post = post or http_utils.post
    outs = []
    for s in samples[:limit]:
        n = int(s.response_length or 0)
        ids = list(s.tokens[:len(s.tokens) - n]) if s.tokens else None
        payload = {"sampling_params": {"max_new_tokens": max_new_tokens, "temperature": temperature}, "return_logprob": False}
        payload.update({"input_ids": ids} if ids else {"text": s.prompt})
        r = await post(url.rstrip("/") + "/generate", payload)
        outs.append(r)
        print(f"--- index={s.index} -> {len(r.get('output_ids', []))} tokens: {_short(r.get('text') or r.get('output_ids'))}", file=out)
    return outs


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m miles_b200.tools.debug_rollout_data")
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("show")
    p.add_argument("path")
    p.add_argument("--limit", type=int, default=8)
    p.add_argument("--tokenizer", default=None)
    p = sub.add_parser("score")
    p.add_argument("path")
    p.add_argument("--rm-type", default=None)
    p.add_argument("--custom-rm-path", default=None)
    p = sub.add_parser("send")
    p.add_argument("path")
    p.add_argument("--url", required=True)
    p.add_argument("--limit", type=int, default=4)
    p.add_argument("--max-new-tokens", type=int, default=64)
    p.add_argument("--temperature", type=float, default=0.0)
    a = ap.parse_args(argv)
    samples = load_samples(a.path)
    if a.cmd == "show":
        tok = None
        if a.tokenizer:
            from transformers import AutoTokenizer

            tok = AutoTokenizer.from_pretrained(a.tokenizer)
        show(samples, a.limit, tok)
    elif a.cmd == "score":
        if not (a.rm_type or a.custom_rm_path):
            ap.error("score needs --rm-type or --custom-rm-path")
        asyncio.run(rescore(samples, a.rm_type, a.custom_rm_path))
    else:
        asyncio.run(send(samples, a.url, a.limit, a.max_new_tokens, a.temperature))
    return 0


if __name__ == "__main__":
    sys.exit(main())
