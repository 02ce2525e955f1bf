"""Train / inference mismatch helper: importance weights between the log-probs the trainer recomputes and the ones the
rollout engine reported, with the usual variance controls, as a plug-in for ``--custom-tis-function-path
miles_b200.rl.mis.mis_function`` (options come from ``--custom-config-path mis.yaml``, see ``examples/train_infer_mismatch``).

* level: ``token`` (per-token ratio), ``sequence`` (product over the sample's trainable tokens), ``geometric`` (its
  geometric mean), each broadcast back onto the sample's tokens;
* mode: ``truncate`` (cap at the upper bound), ``clip`` (into ``[lower, upper]``), ``mask`` (tokens whose weight leaves the
  band drop out of the loss, the others keep their exact weight);
* rejection sampling (``use_rs``): a second band, possibly at another level, that only masks; ``rs_veto_threshold`` drops a
  whole sample when any of its tokens has a ratio below the threshold;
* ``tis_batch_normalize``: divide the weights by their mean over this rank's batch.

Everything works on the packed layout of the loss code: flat ``[tokens]`` tensors plus the sample index of every token, so
per-sample reductions are ``index_add_`` calls and no Python loop runs over samples. Returned metrics are per-token tensors;
the caller reduces them like every other metric (per-sample mean, then mean over samples, or per token).

Reference behaviour: examples/infra_features/train_infer_mismatch_helper/mis.py:151-398 (``compute_mis_weights``), which
loops over per-sample lists.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch

SAFETY_BOUND = 20.0  # |log ratio| is clamped to this before exponentiation


@dataclass
class MisOptions:
    use_tis: bool = True
    tis_level: str = "token"        # token | sequence | geometric
    tis_mode: str = "truncate"      # truncate | clip | mask
    tis_upper_bound: float = 2.0
    tis_lower_bound: Optional[float] = None   # default 1 / upper
    use_rs: bool = False
    rs_level: str = "token"
    rs_lower_bound: Optional[float] = None    # default: the tis bounds
    rs_upper_bound: Optional[float] = None
    rs_veto_threshold: Optional[float] = None
    tis_batch_normalize: bool = False

    @classmethod
    def from_args(cls, args) -> "MisOptions":
        kw = {f: getattr(args, f) for f in cls.__dataclass_fields__ if args is not None and getattr(args, f, None) is not None}
        o = cls(**kw)
        for name, allowed in (("tis_level", ("token", "sequence", "geometric")), ("rs_level", ("token", "sequence", "geometric")),
                              ("tis_mode", ("truncate", "clip", "mask"))):
            if getattr(o, name) not in allowed:
                raise ValueError(f"{name} must be one of {allowed}, got {getattr(o, name)!r}")
        return o


def _per_sample(x: torch.Tensor, mask: torch.Tensor, seg: torch.Tensor, S: int, mean: bool) -> torch.Tensor:
    tot = torch.zeros(S, dtype=torch.float32, device=x.device).index_add_(0, seg, x * mask)
    if mean:
        tot = tot / torch.zeros(S, dtype=torch.float32, device=x.device).index_add_(0, seg, mask).clamp_min(1.0)
    return tot[seg]


def _leveled(log_ratio: torch.Tensor, mask: torch.Tensor, seg: torch.Tensor, S: int, level: str) -> torch.Tensor:
    if level == "token":
        return log_ratio
    return _per_sample(log_ratio, mask, seg, S, mean=(level == "geometric"))


def mis_weights(train_log_probs: torch.Tensor, rollout_log_probs: torch.Tensor, loss_mask: torch.Tensor, seg: torch.Tensor,
                opts: MisOptions, num_samples: Optional[int] = None):
    """Returns ``(weights or None, mask, metrics)``: detached weights to multiply the per-token policy loss with (None
    when ``use_tis`` is off), the loss mask with rejected tokens removed, per-token metric tensors."""
    mask = loss_mask.float()
    seg = seg.long()
    S = int(num_samples if num_samples is not None else (int(seg.max().item()) + 1 if seg.numel() else 0))
    raw = (train_log_probs.float() - rollout_log_probs.float()).detach()
    m: dict = {}
    # how far apart the two engines are, independent of any correction
    m["mismatch_abs_logprob_diff"] = raw.abs()
    m["mismatch_kl_rollout_to_train"] = -raw                      # E_rollout[log p_rollout - log p_train]
    m["mismatch_train_ppl"] = torch.exp(-_per_sample(train_log_probs.float().detach(), mask, seg, S, mean=True))
    m["mismatch_rollout_ppl"] = torch.exp(-_per_sample(rollout_log_probs.float(), mask, seg, S, mean=True))
    lo_t = opts.tis_lower_bound if opts.tis_lower_bound is not None else 1.0 / opts.tis_upper_bound
    new_mask = mask.clone()
    weights = None
    lr_tis = None
    if opts.use_tis:
        lr_tis = _leveled(raw, mask, seg, S, opts.tis_level)
        w = torch.exp(lr_tis.clamp(-SAFETY_BOUND, SAFETY_BOUND))
        m["tis_weight_before_bound"] = w
        if opts.tis_mode == "truncate":
            m["tis_truncate_fraction"] = (w > opts.tis_upper_bound).float()
            w = w.clamp(0.0, opts.tis_upper_bound) * mask
        elif opts.tis_mode == "clip":
            assert lo_t < opts.tis_upper_bound
            m["tis_clip_fraction_low"] = (w < lo_t).float()
            m["tis_clip_fraction_high"] = (w > opts.tis_upper_bound).float()
            w = w.clamp(lo_t, opts.tis_upper_bound) * mask
        else:  # mask: out-of-band tokens leave the loss, in-band tokens keep their exact weight
            m["tis_mask_fraction_low"] = (w < lo_t).float()
            m["tis_mask_fraction_high"] = (w > opts.tis_upper_bound).float()
            new_mask = new_mask * ((w >= lo_t) & (w <= opts.tis_upper_bound)).float()
            w = w * mask
        m["tis_weight_after_bound"] = w
        weights = w
    if opts.use_rs:
        lr_rs = lr_tis if (lr_tis is not None and opts.rs_level == opts.tis_level) else _leveled(raw, mask, seg, S, opts.rs_level)
        r = torch.exp(lr_rs.clamp(-SAFETY_BOUND, SAFETY_BOUND))
        lo = opts.rs_lower_bound if opts.rs_lower_bound is not None else lo_t
        hi = opts.rs_upper_bound if opts.rs_upper_bound is not None else opts.tis_upper_bound
        assert lo < hi
        m["rs_mask_fraction_low"] = (r < lo).float()
        m["rs_mask_fraction_high"] = (r > hi).float()
        new_mask = new_mask * ((r >= lo) & (r <= hi)).float()
        if opts.rs_veto_threshold is not None:
            bad = ((raw < math.log(opts.rs_veto_threshold)) & (mask > 0)).float()
            seq_bad = (torch.zeros(S, dtype=torch.float32, device=raw.device).index_add_(0, seg, bad) > 0).float()[seg]
            m["rs_catastrophic_token_fraction"] = bad
            m["rs_catastrophic_seq_fraction"] = seq_bad
            new_mask = new_mask * (1.0 - seq_bad)
    if weights is not None:
        m["is_ratio_mean_after_tis_rs"] = weights
        if opts.tis_batch_normalize:
            if opts.tis_level == "token":
                mean = (weights * mask).sum() / mask.sum().clamp_min(1.0)
            else:  # one weight per sample: the mean over samples
                per = torch.zeros(S, dtype=torch.float32, device=raw.device).index_add_(0, seg, weights * mask)
                cnt = torch.zeros(S, dtype=torch.float32, device=raw.device).index_add_(0, seg, mask)
                has = cnt > 0
                mean = (per[has] / cnt[has]).mean() if bool(has.any()) else torch.ones((), device=raw.device)
            if float(mean) > 1e-8:
                weights = weights / mean
                m["batch_norm_factor"] = mean.expand_as(weights)
            else:
                m["batch_norm_factor"] = torch.ones_like(weights)
        m["is_ratio_final"] = weights
        weights = weights.detach()
    m["rejected_token_fraction"] = (mask - new_mask).clamp_min(0.0)
    return weights, new_mask.detach(), {k: v.detach() for k, v in m.items()}


def mis_function(cfg, *, pg_loss: torch.Tensor, train_log_probs: torch.Tensor, rollout_log_probs: torch.Tensor,
                 loss_mask: torch.Tensor, seg: torch.Tensor, **_):
    """The ``--custom-tis-function-path`` entry point: ``(pg_loss * weights, new mask, metrics)``. Under context
    parallelism every rank sees its own tokens of a sample: token-level weights are exact there; sequence-level ones use
    the local tokens only (the reference gathers the log-probs over the context-parallel group first)."""
    opts = MisOptions.from_args(getattr(cfg, "args", None))
    weights, new_mask, metrics = mis_weights(train_log_probs, rollout_log_probs, loss_mask, seg, opts)
    if weights is not None and getattr(cfg, "use_tis", True):
        pg_loss = pg_loss * weights
    changed = bool((new_mask != loss_mask.float()).any())
    return pg_loss, (new_mask if changed else None), metrics
