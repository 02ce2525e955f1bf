"""Reward post-processing on the rollout side.

Group normalisation as in miles/ray/rollout/train_data_conversion.py:207-254 of the reference: for
``grpo`` / ``gspo`` / ``reinforce_plus_plus_baseline`` the rewards of one prompt group are centred; for
grpo/gspo they are additionally divided by the unbiased std + 1e-6 when the group has more than one
rollout.  A multi-sample rollout (one trajectory split into several training samples) counts once:
statistics are taken over one reward per *rollout id* and broadcast back to its samples.
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Sequence

import torch

_CENTRED = ("grpo", "gspo", "reinforce_plus_plus_baseline")


def normalize_group_rewards(
    rewards: Sequence[float],
    group_ids: Sequence[int],
    rollout_ids: Sequence[int] | None = None,
    *,
    advantage_estimator: str = "grpo",
    normalize: bool = True,
    std_normalization: bool = True,
) -> list[float]:
    """Return the per-sample normalised rewards (raw rewards are left to the caller for logging)."""
    n = len(rewards)
    if rollout_ids is None:
        rollout_ids = list(range(n))
    if not normalize or advantage_estimator not in _CENTRED:
        return [float(r) for r in rewards]
    groups: "OrderedDict[int, OrderedDict[int, float]]" = OrderedDict()
    for r, g, rid in zip(rewards, group_ids, rollout_ids):
        d = groups.setdefault(g, OrderedDict())
        if rid in d:
            if abs(d[rid] - float(r)) > 1e-8:
                raise ValueError(f"samples of rollout {rid} carry different rewards ({d[rid]} vs {r})")
        else:
            d[rid] = float(r)
    out_by_rollout: dict[tuple[int, int], float] = {}
    for g, d in groups.items():
        vals = torch.tensor(list(d.values()), dtype=torch.float64)
        centred = vals - vals.mean()
        if advantage_estimator in ("grpo", "gspo") and std_normalization and len(vals) > 1:
            std = vals.std(unbiased=True)
            if float(std) > 0:
                centred = centred / (std + 1e-6)
        for rid, v in zip(d.keys(), centred.tolist()):
            out_by_rollout[(g, rid)] = v
    return [out_by_rollout[(g, rid)] for g, rid in zip(group_ids, rollout_ids)]
