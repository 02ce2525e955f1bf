"""Policy / value / SFT losses over flat packed response tokens.

Semantics follow miles/backends/training_utils/loss_hub/losses.py:62-519 and
loss_hub/math_utils.py:183-277 of the reference: PPO ratio from ``ppo_kl = logp_old - logp_new`` with
the exponent clamped, clip ``[1-eps, 1+eps_high]`` and optional dual clip, GSPO sequence-level KL,
OPSM sequence masking, TIS / ICEPOP off-policy corrections, entropy bonus, KL-to-reference loss, and
the same metric names.  The implementation is vectorised: every per-sample quantity is a segment
reduction over ``seg`` (token -> sample index), so there is no Python loop over samples.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch

from .kl import compute_approx_kl, safe_exp_neg


@dataclass
class LossConfig:
    advantage_estimator: str = "grpo"
    eps_clip: float = 0.2
    eps_clip_high: float = 0.2
    eps_clip_c: Optional[float] = None
    entropy_coef: float = 0.0
    observe_training_entropy: bool = False
    use_kl_loss: bool = False
    kl_loss_coef: float = 0.0
    kl_loss_type: str = "k1"
    use_unbiased_kl: bool = False
    use_rollout_logprobs: bool = False
    use_tis: bool = False
    tis_mode: str = "tis"  # "tis" (clamp) | "icepop" (zero outside the band)
    tis_clip: float = 2.0
    tis_clip_low: float = 0.0
    get_mismatch_metrics: bool = False
    use_opsm: bool = False
    opsm_delta: float = 1e-4
    calculate_per_token_loss: bool = False
    value_clip: float = 0.2
    custom_tis_fn: Optional[Callable] = None
    custom_pg_reducer_fn: Optional[Callable] = None

    @classmethod
    def from_args(cls, args) -> "LossConfig":
        kw = {}
        for f in cls.__dataclass_fields__:
            if hasattr(args, f) and getattr(args, f) is not None:
                kw[f] = getattr(args, f)
        cfg = cls(**kw)
        if getattr(args, "eps_clip_high", None) is None:
            cfg.eps_clip_high = cfg.eps_clip
        return cfg


class SegmentReducer:
    """``sum_s (sum_{t in s} x_t m_t) / denom_s`` — per-sample mean, summed over samples.

    ``denoms`` are the trainable-token counts of the *whole rollout* a sample belongs to
    (``rollout_mask_sums``), so a trajectory split into several samples counts once.  With
    ``per_token`` the plain masked sum is returned and the caller normalises by the token count.
    """

    def __init__(self, seg: torch.Tensor, mask: torch.Tensor, denoms: Optional[torch.Tensor] = None,
                 per_token: bool = False, num_samples: Optional[int] = None):
        self.seg = seg
        self.mask = mask.float()
        S = int(num_samples if num_samples is not None else (int(seg.max().item()) + 1 if seg.numel() else 0))
        self.num_samples = S
        if denoms is None:
            denoms = torch.zeros(S, dtype=torch.float32, device=mask.device).index_add_(0, seg, self.mask)
        self.denoms = denoms.float().clamp_min(1.0)
        self.per_token = per_token
        self._w = self.mask if per_token else self.mask / self.denoms[seg] if seg.numel() else self.mask

    def with_mask(self, mask: torch.Tensor) -> "SegmentReducer":
        r = SegmentReducer.__new__(SegmentReducer)
        r.seg, r.mask, r.denoms, r.per_token, r.num_samples = self.seg, mask.float(), self.denoms, self.per_token, self.num_samples
        r._w = r.mask if r.per_token else (r.mask / r.denoms[r.seg] if r.seg.numel() else r.mask)
        return r

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        return (x * self._w).sum()

    def seq_mean(self, x: torch.Tensor) -> torch.Tensor:
        """Masked mean of x within each sample (own token count as denominator) -> [S]."""
        num = torch.zeros(self.num_samples, dtype=torch.float32, device=x.device).index_add_(0, self.seg, x.float() * self.mask)
        den = torch.zeros(self.num_samples, dtype=torch.float32, device=x.device).index_add_(0, self.seg, self.mask)
        return num / den.clamp_min(1.0)


def _clean(x: torch.Tensor, active: torch.Tensor) -> torch.Tensor:
    return torch.where(active, torch.nan_to_num(x, nan=0.0, posinf=0.0, neginf=0.0), torch.zeros((), dtype=x.dtype, device=x.device))


def compute_policy_loss(ppo_kl, advantages, eps_clip, eps_clip_high, eps_clip_c=None):
    ratio = safe_exp_neg(ppo_kl)
    l1 = -ratio * advantages
    l2 = -ratio.clamp(1 - eps_clip, 1 + eps_clip_high) * advantages
    clipped = torch.maximum(l1, l2)
    clipfrac = (l2 > l1).float()
    if eps_clip_c is not None:
        assert eps_clip_c > 1.0, "the dual-clip constant must exceed 1"
        l3 = -eps_clip_c * advantages
        clipped = torch.where(advantages < 0, torch.minimum(l3, clipped), clipped)
    return clipped, clipfrac


def policy_loss(
    cfg: LossConfig,
    log_probs: torch.Tensor,
    entropy: Optional[torch.Tensor],
    *,
    old_log_probs: Optional[torch.Tensor],
    advantages: torch.Tensor,
    reducer: SegmentReducer,
    rollout_log_probs: Optional[torch.Tensor] = None,
    ref_log_probs: Optional[torch.Tensor] = None,
    opd_reverse_kl: Optional[torch.Tensor] = None,
):
    """Returns ``(loss, metrics)``; ``loss`` is the un-rescaled sum over local samples."""
    seg, mask = reducer.seg, reducer.mask
    active = mask.bool()
    log_probs = log_probs.float()
    if cfg.use_rollout_logprobs:
        assert rollout_log_probs is not None, "rollout log-probs are required by use_rollout_logprobs"
        old = rollout_log_probs.float().detach()
        trainer_old = old_log_probs.float().detach() if old_log_probs is not None else None
    else:
        old = (old_log_probs.float() if old_log_probs is not None else log_probs).detach()
        trainer_old = old
    adv = _clean(advantages.float().detach(), active)

    if cfg.use_opsm or cfg.advantage_estimator == "gspo":
        seq_kl = reducer.seq_mean(old - log_probs)  # [S], differentiable for GSPO
    opsm_mask = None
    metrics: dict[str, torch.Tensor] = {}
    if cfg.use_opsm:
        with torch.no_grad():
            drop = (adv < 0) & (seq_kl.detach()[seg] > cfg.opsm_delta)
            opsm_mask = 1.0 - drop.float()
            counts = torch.zeros(reducer.num_samples, device=mask.device).index_add_(0, seg, mask)
            # per sample: dropped tokens over trainable tokens, summed over samples (the reference counts every token of a
            # dropped sequence in the numerator, miles/backends/training_utils/loss_hub/math_utils.py:182-222)
            metrics["opsm_clipfrac"] = (drop.float() / counts.clamp_min(1.0)[seg]).sum()

    if cfg.advantage_estimator == "gspo":
        ppo_kl = seq_kl[seg]
    else:
        ppo_kl = old - log_probs
    ppo_kl = _clean(ppo_kl, active)

    pg, clipfrac = compute_policy_loss(ppo_kl, adv, cfg.eps_clip, cfg.eps_clip_high, cfg.eps_clip_c)
    if opsm_mask is not None:
        pg = pg * opsm_mask

    pg_reducer = reducer
    tis_metrics = {}
    if cfg.use_tis or cfg.get_mismatch_metrics:
        assert rollout_log_probs is not None and trainer_old is not None, "TIS needs trainer and rollout log-probs"
        ois = torch.exp(-ppo_kl.detach())
        if cfg.custom_tis_fn is not None:
            pg, new_mask, tis_metrics = cfg.custom_tis_fn(cfg, pg_loss=pg, train_log_probs=trainer_old,
                                                          rollout_log_probs=rollout_log_probs.float(), loss_mask=mask, seg=seg)
            if new_mask is not None:
                pg_reducer = reducer.with_mask(new_mask)
        else:
            ratio = torch.exp(trainer_old - rollout_log_probs.float())
            if cfg.tis_mode == "icepop":
                wts = torch.where((ratio >= cfg.tis_clip_low) & (ratio <= cfg.tis_clip), ratio, torch.zeros_like(ratio))
            else:
                wts = ratio.clamp(min=cfg.tis_clip_low, max=cfg.tis_clip)
            tis_metrics = {"tis": ratio.detach(), "tis_clipfrac": (wts != ratio).float(), "tis_abs": (ratio - 1).abs().detach()}
            if cfg.use_tis:
                pg = pg * wts.detach()
        metrics["ois"] = reducer(ois).detach()
        for k, v in tis_metrics.items():
            metrics[k] = reducer(v.float()).detach()
    if cfg.custom_pg_reducer_fn is not None:
        pg_reducer = cfg.custom_pg_reducer_fn(reducer)

    # effective-sample-size ratio of the per-token importance weights, per sample
    with torch.no_grad():
        wts = safe_exp_neg(ppo_kl.detach()) * mask
        S = reducer.num_samples
        sw = torch.zeros(S, device=mask.device).index_add_(0, seg, wts)
        sw2 = torch.zeros(S, device=mask.device).index_add_(0, seg, wts * wts)
        n = torch.zeros(S, device=mask.device).index_add_(0, seg, mask).clamp_min(1.0)
        ess = (sw * sw) / (n * sw2.clamp_min(1e-8))
        has = torch.zeros(S, device=mask.device).index_add_(0, seg, torch.ones_like(mask)) > 0
        metrics["ess_ratio"] = ((ess * n) if cfg.calculate_per_token_loss else ess)[has].sum()

    pg_loss = pg_reducer(pg)
    loss = pg_loss
    entropy_loss = torch.zeros((), device=mask.device)
    if entropy is not None and (cfg.entropy_coef != 0 or cfg.observe_training_entropy):
        entropy_loss = reducer(entropy.float())
        if cfg.entropy_coef != 0:
            loss = loss - cfg.entropy_coef * entropy_loss
        else:
            entropy_loss = entropy_loss.detach()

    if cfg.use_kl_loss:
        assert ref_log_probs is not None, "ref log-probs are required by use_kl_loss"
        ir = torch.exp(log_probs - old) if cfg.use_unbiased_kl else None
        kl = _clean(compute_approx_kl(log_probs, ref_log_probs.float(), cfg.kl_loss_type, ir), active)
        kl_loss = reducer(kl)
        if cfg.kl_loss_coef != 0:
            loss = loss + cfg.kl_loss_coef * kl_loss
        metrics["kl_loss"] = kl_loss.detach()

    if log_probs.numel() == 0:
        loss = loss + 0.0 * log_probs.sum()

    metrics.update({
        "loss": loss.detach(),
        "pg_loss": pg_loss.detach(),
        "entropy_loss": entropy_loss.detach(),
        "pg_clipfrac": reducer(clipfrac).detach(),
        "ppo_kl": reducer(ppo_kl.detach()).detach(),
    })
    if rollout_log_probs is not None and trainer_old is not None:
        rl = rollout_log_probs.float()
        metrics["train_rollout_logprob_abs_diff"] = reducer(_clean((trainer_old - rl).abs(), active)).detach()
        metrics["train_rollout_kl"] = reducer(_clean(compute_approx_kl(rl, trainer_old, "low_var_kl"), active)).detach()
    if opd_reverse_kl is not None:
        metrics["opd_reverse_kl"] = reducer(opd_reverse_kl.float()).detach()
    return loss, metrics


def value_loss(cfg: LossConfig, values: torch.Tensor, *, old_values: torch.Tensor, returns: torch.Tensor,
               reducer: SegmentReducer):
    values = values.float()
    old_values, returns = old_values.float().detach(), returns.float().detach()
    clipfrac = ((values - old_values).abs() > cfg.value_clip).float()
    clipped = old_values + (values - old_values).clamp(-cfg.value_clip, cfg.value_clip)
    loss = reducer(torch.maximum((clipped - returns) ** 2, (values - returns) ** 2))
    if values.numel() == 0:
        loss = loss + 0.0 * values.sum()
    return loss, {"value_loss": loss.detach(), "value_clipfrac": reducer(clipfrac).detach()}


def sft_loss(cfg: LossConfig, log_probs: torch.Tensor, *, reducer: SegmentReducer):
    loss = -reducer(log_probs.float())
    if log_probs.numel() == 0:
        loss = loss + 0.0 * log_probs.sum()
    return loss, {"loss": loss.detach()}
