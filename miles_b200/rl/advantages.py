"""Advantage estimators over flat packed response tokens.

Inputs are 1-D tensors over the response-aligned tokens of all local samples plus ``cu`` (int64
``[S+1]`` cumulative response lengths).  Estimators (behaviour of
miles/backends/training_utils/loss_hub/advantages.py:16-105 in the reference):

* ``grpo`` / ``gspo``: the (group-normalised) scalar reward is broadcast to every token.
* ``ppo``: token reward ``-kl_coef * KL_t``, the scalar reward is added at the last *trainable*
  token, GAE(gamma, lambda) runs over trainable tokens only (masked tool/observation tokens are not
  MDP steps), returns = advantages + values.
* ``reinforce_plus_plus``: discounted return of the same token rewards.
* ``reinforce_plus_plus_baseline``: ``A_t = r - kl_coef * KL_t``.

GAE is evaluated with the chunked formulation (one GEMM against a 128x128 power matrix for all
chunks, then a short sequential carry across chunks), on the GPU through ``ops.gae`` when available.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from .kl import compute_approx_kl


def seg_ids(cu: torch.Tensor) -> torch.Tensor:
    """Token -> sample index for cumulative lengths ``cu`` ([S+1])."""
    lens = (cu[1:] - cu[:-1]).to(torch.long)
    return torch.repeat_interleave(torch.arange(lens.numel(), device=cu.device), lens)


def vanilla_gae(rewards: torch.Tensor, values: torch.Tensor, gamma: float, lam: float):
    """Reference loop. rewards/values: [B, T]; returns (advantages, returns)."""
    B, T = rewards.shape
    adv = torch.zeros_like(rewards)
    last = torch.zeros(B, dtype=rewards.dtype, device=rewards.device)
    for t in reversed(range(T)):
        nxt = values[:, t + 1] if t + 1 < T else torch.zeros_like(last)
        delta = rewards[:, t] + gamma * nxt - values[:, t]
        last = delta + gamma * lam * last
        adv[:, t] = last
    return adv, adv + values


def chunked_gae(rewards: torch.Tensor, values: torch.Tensor, gamma: float, lam: float, chunk: int = 128):
    """Chunk-parallel GAE on padded [B, T] inputs (padding must be zero rewards and values at the tail).

    On the time-reversed sequence ``A'_j = x_j + w A'_{j-1}`` with ``w = gamma*lambda``; within a chunk
    ``A' = x @ M + w^(j+1) * carry`` where ``M[i, j] = w^(j-i)`` for ``j >= i``.
    """
    B, T = rewards.shape
    dtype = torch.float32
    r = rewards.to(dtype)
    v = values.to(dtype)
    nxt = torch.cat([v[:, 1:], torch.zeros(B, 1, dtype=dtype, device=v.device)], dim=1)
    delta = r + gamma * nxt - v
    w = gamma * lam
    x = delta.flip(1)
    pad = (-T) % chunk
    if pad:
        x = torch.cat([x, torch.zeros(B, pad, dtype=dtype, device=x.device)], dim=1)
    n = x.shape[1] // chunk
    xc = x.view(B, n, chunk)
    idx = torch.arange(chunk, device=x.device)
    expo = (idx[None, :] - idx[:, None]).to(dtype)
    M = torch.where(expo >= 0, torch.pow(torch.tensor(w, dtype=dtype, device=x.device), expo.clamp(min=0)),
                    torch.zeros((), dtype=dtype, device=x.device))
    local = xc @ M  # [B, n, chunk]
    pw = torch.pow(torch.tensor(w, dtype=dtype, device=x.device), (idx + 1).to(dtype))  # w^(j+1)
    out = torch.empty_like(local)
    carry = torch.zeros(B, dtype=dtype, device=x.device)
    for c in range(n):
        out[:, c] = local[:, c] + carry[:, None] * pw[None, :]
        carry = out[:, c, -1]
    adv = out.view(B, n * chunk)[:, :T].flip(1)
    return adv.to(rewards.dtype), (adv + v).to(rewards.dtype)


def _pad_segments(x: torch.Tensor, cu: torch.Tensor):
    """Flat [N] + cu [S+1] -> padded [S, Tmax] (zeros) and the boolean validity mask."""
    lens = (cu[1:] - cu[:-1]).to(torch.long)
    S = lens.numel()
    tmax = int(lens.max().item()) if S > 0 else 0
    pos = torch.arange(tmax, device=x.device)[None, :]
    valid = pos < lens[:, None]
    out = torch.zeros(S, tmax, dtype=x.dtype, device=x.device)
    out[valid] = x
    return out, valid


def gae_flat(token_rewards: torch.Tensor, values: torch.Tensor, mask: torch.Tensor, cu: torch.Tensor,
             gamma: float, lam: float, chunked: bool = True):
    """GAE over the trainable tokens of each segment; non-trainable positions get zero advantage."""
    m = mask.bool()
    seg = seg_ids(cu)
    S = cu.numel() - 1
    kept_counts = torch.zeros(S, dtype=torch.long, device=cu.device).index_add_(0, seg[m], torch.ones_like(seg[m]))
    cu_kept = torch.cat([torch.zeros(1, dtype=torch.long, device=cu.device), kept_counts.cumsum(0)])
    r_k, v_k = token_rewards[m].float(), values[m].float()
    if r_k.numel() == 0:
        z = torch.zeros_like(token_rewards, dtype=torch.float32)
        return z, z.clone()
    rp, valid = _pad_segments(r_k, cu_kept)
    vp, _ = _pad_segments(v_k, cu_kept)
    fn = chunked_gae if chunked else vanilla_gae
    ap, retp = fn(rp, vp, gamma, lam)
    adv = torch.zeros_like(token_rewards, dtype=torch.float32)
    ret = torch.zeros_like(token_rewards, dtype=torch.float32)
    adv[m] = ap[valid]
    ret[m] = retp[valid]
    return adv, ret


def last_trainable_index(mask: torch.Tensor, cu: torch.Tensor) -> torch.Tensor:
    """Flat index of the last token with mask==1 in each segment (-1 when a segment has none)."""
    seg = seg_ids(cu)
    S = cu.numel() - 1
    pos = torch.arange(mask.numel(), device=mask.device)
    cand = torch.where(mask.bool(), pos, torch.full_like(pos, -1))
    out = torch.full((S,), -1, dtype=torch.long, device=mask.device)
    return out.scatter_reduce(0, seg, cand, reduce="amax", include_self=True)


def discounted_returns_flat(token_rewards: torch.Tensor, cu: torch.Tensor, gamma: float) -> torch.Tensor:
    """G_t = r_t + gamma G_{t+1} within each segment (all positions are steps)."""
    ones = torch.ones_like(token_rewards, dtype=torch.float32)
    zeros = torch.zeros_like(ones)
    adv, _ = gae_flat(token_rewards.float(), zeros, ones, cu, gamma, 1.0)
    return adv


def whiten(values: torch.Tensor, mask: torch.Tensor, group: Optional["dist.ProcessGroup"] = None,
           shift_mean: bool = True, eps: float = 1e-8, reduce: bool = True) -> torch.Tensor:
    """Masked whitening with statistics all-reduced over ``group`` (3 floats), Bessel-corrected."""
    m = mask.to(values.dtype)
    stats = torch.stack([(values * m).sum(), (values * values * m).sum(), m.sum()]).float()
    if reduce and dist.is_available() and dist.is_initialized():
        dist.all_reduce(stats, op=dist.ReduceOp.SUM, group=group)
    s, ss, n = stats[0], stats[1], stats[2]
    if float(n) == 0:
        raise ValueError("whitening over an empty mask")
    mean = s / n
    var = ss / n - mean * mean
    if float(n) >= 2:
        var = var * (n / (n - 1))
    out = (values - mean) * torch.rsqrt(var + eps)
    if not shift_mean:
        out = out + mean
    return out


def compute_advantages_and_returns(
    *,
    advantage_estimator: str,
    rewards: torch.Tensor,
    cu: torch.Tensor,
    loss_mask: torch.Tensor,
    log_probs: Optional[torch.Tensor] = None,
    ref_log_probs: Optional[torch.Tensor] = None,
    values: Optional[torch.Tensor] = None,
    teacher_log_probs: Optional[torch.Tensor] = None,
    kl_coef: float = 0.0,
    kl_loss_type: str = "k1",
    gamma: float = 1.0,
    lambd: float = 1.0,
    normalize_advantages: bool = False,
    opd_kl_coef: float = 0.0,
    dp_group: Optional["dist.ProcessGroup"] = None,
):
    """Return ``(advantages, returns, kl)`` as flat fp32 tensors aligned with ``loss_mask``."""
    N = loss_mask.numel()
    dev = loss_mask.device
    seg = seg_ids(cu)
    rewards = rewards.to(device=dev, dtype=torch.float32)
    if kl_coef == 0 or log_probs is None or ref_log_probs is None:
        kl = torch.zeros(N, dtype=torch.float32, device=dev)
    else:
        kl = compute_approx_kl(log_probs, ref_log_probs, kl_loss_type)

    if advantage_estimator in ("grpo", "gspo"):
        adv = rewards[seg].clone()
        ret = adv.clone()
    elif advantage_estimator == "ppo":
        if values is None:
            raise ValueError("ppo needs critic values")
        tok_r = -kl_coef * kl
        last = last_trainable_index(loss_mask, cu)
        ok = last >= 0
        tok_r = tok_r.index_put((last[ok],), rewards[ok], accumulate=True)
        adv, ret = gae_flat(tok_r, values.float(), loss_mask, cu, gamma, lambd)
    elif advantage_estimator == "reinforce_plus_plus":
        tok_r = -kl_coef * kl
        last = last_trainable_index(loss_mask, cu)
        if bool((last < 0).any()):
            raise ValueError("a sequence is fully masked")
        tok_r = tok_r.index_put((last,), rewards, accumulate=True)
        adv = discounted_returns_flat(tok_r, cu, gamma)
        ret = adv.clone()
    elif advantage_estimator == "reinforce_plus_plus_baseline":
        adv = rewards[seg] - kl_coef * kl
        ret = adv.clone()
    else:
        raise NotImplementedError(f"advantage_estimator {advantage_estimator!r} is not supported")

    if opd_kl_coef != 0.0 and teacher_log_probs is not None and log_probs is not None:
        # on-policy distillation: penalise the student's excess log-prob over the teacher's
        adv = adv - opd_kl_coef * (log_probs.float() - teacher_log_probs.float())

    if normalize_advantages:
        adv = whiten(adv, loss_mask, dp_group)
    return adv, ret, kl
