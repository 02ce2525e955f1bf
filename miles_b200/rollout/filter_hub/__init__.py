"""Dynamic sampling filters (``--dynamic-sampling-filter-path``) and sample filters.

A dynamic filter receives ``(args, group)`` and returns a ``DynamicFilterOutput``; groups that are not
kept are discarded and replaced by over-sampled ones (reference: miles/rollout/filter_hub/)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch


@dataclass
class DynamicFilterOutput:
    keep: bool
    reason: Optional[str] = None


def check_reward_nonzero_std(args, samples, **kwargs) -> DynamicFilterOutput:
    """DAPO-style filter: keep a group only when its rewards are not all equal."""
    key = getattr(args, "reward_key", None)
    rewards = torch.tensor([s.get_reward_value(key) for s in samples], dtype=torch.float64)
    keep = bool(rewards.std(unbiased=False) > 0) if rewards.numel() > 1 else True
    return DynamicFilterOutput(keep, None if keep else f"zero_std_{rewards[0].item():g}")


def check_no_aborted(args, samples, **kwargs) -> DynamicFilterOutput:
    from ...utils.types import Sample

    bad = any(s.status == Sample.Status.ABORTED for s in samples)
    return DynamicFilterOutput(not bad, "aborted" if bad else None)
