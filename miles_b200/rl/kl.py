"""KL estimators between two log-probability vectors.

Behaviour follows miles/backends/training_utils/loss_hub/math_utils.py:138-180 of the reference:
``k1 = d``, ``k2 = d^2/2``, ``k3 = exp(-d) - 1 + d`` with ``d = logp - logp_base`` in fp32;
``low_var_kl`` is k3 with the exponent argument clamped to a safe range and the result clamped to
[-10, 10]; an optional importance ratio multiplies the estimate (unbiased KL).
"""
from __future__ import annotations

import torch

_SAFE_LOG_RATIO = 20.0


def safe_exp_neg(x: torch.Tensor) -> torch.Tensor:
    """exp(-x) with the exponent clamped to +-20 so that a stray token cannot overflow the ratio."""
    return torch.exp(torch.clamp(-x, min=-_SAFE_LOG_RATIO, max=_SAFE_LOG_RATIO))


def compute_approx_kl(
    log_probs: torch.Tensor,
    log_probs_base: torch.Tensor,
    kl_loss_type: str = "k1",
    importance_ratio: torch.Tensor | None = None,
) -> torch.Tensor:
    d = log_probs.float() - log_probs_base.float()
    if kl_loss_type == "k1":
        kl = d
    elif kl_loss_type == "k2":
        kl = 0.5 * d * d
    elif kl_loss_type in ("k3", "low_var_kl"):
        nd = -d
        if kl_loss_type == "low_var_kl":
            nd = torch.clamp(nd, min=-_SAFE_LOG_RATIO, max=_SAFE_LOG_RATIO)
        kl = torch.exp(nd) - 1.0 - nd
    else:
        raise ValueError(f"unknown kl_loss_type {kl_loss_type!r}")
    if importance_ratio is not None:
        kl = importance_ratio * kl
    if kl_loss_type == "low_var_kl":
        kl = torch.clamp(kl, min=-10.0, max=10.0)
    return kl
