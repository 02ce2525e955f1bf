"""On-policy distillation: the student's advantages are lowered by how much more likely it finds its own sampled
token than the teacher does, ``adv -= opd_kl_coef * (student_logprob - teacher_logprob)`` per response token (a
per-token reverse-KL estimate on the student's samples). Teacher log-probs come either from a teacher copy of the
weights scored by the trainer (``teacher`` weight tag) or from an external scoring engine, which may return only
its top-k log-probs per position: tokens outside the teacher's top-k get the floor ``log(remaining mass / (V - k))``.

Reference: miles/backends/training_utils/loss_hub/opd.py:8-94, miles/rollout/on_policy_distillation.py:281-436.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence

import torch


def apply_opd(advantages: torch.Tensor, student_log_probs: torch.Tensor, teacher_log_probs: torch.Tensor,
              opd_kl_coef: float, loss_mask: Optional[torch.Tensor] = None, clip: Optional[float] = None) -> tuple:
    """Returns (new advantages, mean reverse-KL estimate over the trained tokens)."""
    diff = (student_log_probs - teacher_log_probs).detach()
    if clip is not None:
        diff = diff.clamp(-clip, clip)
    out = advantages - opd_kl_coef * diff
    if loss_mask is not None:
        m = loss_mask.to(diff.dtype)
        kl = (diff * m).sum() / m.sum().clamp(min=1.0)
    else:
        kl = diff.mean() if diff.numel() else diff.sum()
    return out, kl


def teacher_logprob_from_topk(token: int, topk_ids: Sequence[int], topk_logprobs: Sequence[float], vocab_size: int) -> float:
    """Log-prob the teacher gives to ``token`` when only its top-k is known."""
    for i, t in enumerate(topk_ids):
        if int(t) == int(token):
            return float(topk_logprobs[i])
    mass = 1.0 - sum(math.exp(float(l)) for l in topk_logprobs)
    rest = max(vocab_size - len(topk_ids), 1)
    return math.log(max(mass, 1e-10) / rest)


def teacher_logprobs_for_sample(tokens: Sequence[int], per_position_topk: Sequence[dict], vocab_size: int) -> list:
    """``per_position_topk[i] = {"ids": [...], "logprobs": [...]}`` for response position ``i``."""
    return [teacher_logprob_from_topk(t, p["ids"], p["logprobs"], vocab_size) for t, p in zip(tokens, per_position_topk)]
