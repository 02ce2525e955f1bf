"""Reads the rollout dumps of a run (``--save-debug-rollout-data`` / ``--dump-details``: one ``{rollout_id}.pt`` per
rollout with every sample as a dict) for the dashboard's rollout inspector: per-rollout summaries, prompt groups,
per-sample token tables with log-probs and loss masks, and the conversation of a sample where one was recorded.

Reference counterpart: miles/dashboard/dump_reader.py (the dashboard reads the same debug dumps the trainer can replay
with ``--load-debug-rollout-data``).
"""
from __future__ import annotations

import os
import re
from typing import Optional

import torch


class DumpReader:
    def __init__(self, directory: str, tokenizer=None, cache: int = 4):
        self.dir, self.tokenizer, self._cache_n = directory, tokenizer, cache
        self._cache: dict = {}

    def rollout_ids(self) -> list:
        if not os.path.isdir(self.dir):
            return []
        ids = []
        for f in os.listdir(self.dir):
            m = re.fullmatch(r"(-?\d+)\.pt", f)
            if m:
                ids.append(int(m.group(1)))
        return sorted(ids)

    def _load(self, rollout_id: int) -> Optional[list]:
        if rollout_id in self._cache:
            return self._cache[rollout_id]
        p = os.path.join(self.dir, f"{rollout_id}.pt")
        if not os.path.exists(p):
            return None
        samples = torch.load(p, weights_only=False)["samples"]
        if len(self._cache) >= self._cache_n:
            self._cache.pop(next(iter(self._cache)))
        self._cache[rollout_id] = samples
        return samples

    @staticmethod
    def _reward(s: dict) -> Optional[float]:
        r = s.get("reward")
        if isinstance(r, dict):
            r = r.get("score", r.get("reward"))
        return float(r) if isinstance(r, (int, float)) else None

    def summary(self, rollout_id: int) -> Optional[dict]:
        samples = self._load(rollout_id)
        if samples is None:
            return None
        rewards = [r for r in (self._reward(s) for s in samples) if r is not None]
        lens = [int(s.get("response_length") or 0) for s in samples]
        status = {}
        for s in samples:
            status[str(s.get("status"))] = status.get(str(s.get("status")), 0) + 1
        versions = sorted({v for s in samples for v in (s.get("weight_versions") or [])})
        return {"rollout_id": rollout_id, "num_samples": len(samples), "num_groups": len({s.get("group_index") for s in samples}),
                "reward_mean": sum(rewards) / len(rewards) if rewards else None,
                "reward_min": min(rewards) if rewards else None, "reward_max": max(rewards) if rewards else None,
                "response_len_mean": sum(lens) / len(lens) if lens else 0, "response_len_max": max(lens) if lens else 0,
                "status": status, "weight_versions": versions,
                "cached_tokens": sum((s.get("prefix_cache_info") or {}).get("cached_tokens", 0) for s in samples)}

    def groups(self, rollout_id: int) -> Optional[list]:
        """One row per prompt group: its samples' rewards and lengths (what GRPO normalises over)."""
        samples = self._load(rollout_id)
        if samples is None:
            return None
        by: dict = {}
        for i, s in enumerate(samples):
            by.setdefault(s.get("group_index"), []).append((i, s))
        out = []
        for g, rows in sorted(by.items(), key=lambda kv: (kv[0] is None, kv[0])):
            rs = [self._reward(s) for _, s in rows]
            known = [r for r in rs if r is not None]
            mean = sum(known) / len(known) if known else None
            out.append({"group_index": g, "samples": [i for i, _ in rows], "rewards": rs,
                        "reward_mean": mean, "reward_std": (sum((r - mean) ** 2 for r in known) / len(known)) ** 0.5 if known else None,
                        "response_lengths": [int(s.get("response_length") or 0) for _, s in rows],
                        "all_equal": len(set(known)) <= 1})   # a group without reward variance gives GRPO no signal
        return out

    def sample_tokens(self, rollout_id: int, index: int) -> Optional[dict]:
        samples = self._load(rollout_id)
        if samples is None or not 0 <= index < len(samples):
            return None
        s = samples[index]
        toks = list(s.get("tokens") or [])
        n = int(s.get("response_length") or 0)
        resp = toks[len(toks) - n:] if n else []
        lps = list(s.get("rollout_log_probs") or [])
        mask = list(s.get("loss_mask") or [1] * n)
        text = [self.tokenizer.decode([t]) for t in resp] if self.tokenizer is not None else None
        return {"rollout_id": rollout_id, "index": index, "prompt_tokens": len(toks) - n, "response_tokens": n,
                "reward": self._reward(s), "status": str(s.get("status")),
                "tokens": [{"id": int(t), "text": text[j] if text else None, "logprob": float(lps[j]) if j < len(lps) else None,
                            "loss_mask": int(mask[j]) if j < len(mask) else 1} for j, t in enumerate(resp)]}

    def sample_messages(self, rollout_id: int, index: int) -> Optional[dict]:
        samples = self._load(rollout_id)
        if samples is None or not 0 <= index < len(samples):
            return None
        s = samples[index]
        msgs = (s.get("metadata") or {}).get("messages")
        if not msgs:
            prompt = s.get("prompt")
            msgs = (prompt if isinstance(prompt, list) and prompt and isinstance(prompt[0], dict) else
                    [{"role": "user", "content": prompt if isinstance(prompt, str) else f"<{len(s.get('tokens') or []) - int(s.get('response_length') or 0)} prompt tokens>"}])
            msgs = list(msgs) + [{"role": "assistant", "content": s.get("response") or ""}]
        return {"rollout_id": rollout_id, "index": index, "messages": msgs, "reward": self._reward(s), "label": s.get("label")}
