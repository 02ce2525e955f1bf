"""Train / inference mismatch helper (rl/mis.py) against a per-sample loop written the obvious way, and inside the policy
loss through --custom-tis-function-path."""
import math
from types import SimpleNamespace

import pytest
import torch

from miles_b200.rl.mis import MisOptions, mis_function, mis_weights


def _batch(seed=0, lens=(5, 1, 9, 4)):
    g = torch.Generator().manual_seed(seed)
    seg = torch.cat([torch.full((n,), i) for i, n in enumerate(lens)])
    T = seg.numel()
    train = -torch.rand(T, generator=g) * 2
    rollout = train + torch.randn(T, generator=g) * 0.4
    mask = (torch.rand(T, generator=g) > 0.25).float()
    mask[5] = 1.0  # the one-token sample stays trainable
    return train, rollout, mask, seg, len(lens)


def _oracle(train, rollout, mask, seg, S, o: MisOptions):
    """Per-sample loop; returns (weights, new_mask)."""
    W, M = torch.zeros_like(train), mask.clone()
    lo_t = o.tis_lower_bound if o.tis_lower_bound is not None else 1.0 / o.tis_upper_bound

    def level(raw, m, kind):
        if kind == "token":
            return raw
        tot = (raw * m).sum()
        return (tot / m.sum().clamp_min(1) if kind == "geometric" else tot).expand_as(raw)

    for s in range(S):
        idx = (seg == s).nonzero().flatten()
        raw, m = (train - rollout)[idx], mask[idx]
        nm = m.clone()
        w = torch.ones_like(raw)
        if o.use_tis:
            w = torch.exp(level(raw, m, o.tis_level).clamp(-20, 20))
            if o.tis_mode == "truncate":
                w = w.clamp(0, o.tis_upper_bound) * m
            elif o.tis_mode == "clip":
                w = w.clamp(lo_t, o.tis_upper_bound) * m
            else:
                nm = nm * ((w >= lo_t) & (w <= o.tis_upper_bound)).float()
                w = w * m
        if o.use_rs:
            r = torch.exp(level(raw, m, o.rs_level).clamp(-20, 20))
            lo = o.rs_lower_bound if o.rs_lower_bound is not None else lo_t
            hi = o.rs_upper_bound if o.rs_upper_bound is not None else o.tis_upper_bound
            nm = nm * ((r >= lo) & (r <= hi)).float()
            if o.rs_veto_threshold is not None and bool(((raw < math.log(o.rs_veto_threshold)) & (m > 0)).any()):
                nm = nm * 0
        W[idx], M[idx] = w, nm
    return W, M


@pytest.mark.parametrize("opts", [
    MisOptions(tis_level="token", tis_mode="truncate", tis_upper_bound=1.5),
    MisOptions(tis_level="sequence", tis_mode="clip", tis_upper_bound=2.0, tis_lower_bound=0.7),
    MisOptions(tis_level="geometric", tis_mode="mask", tis_upper_bound=1.2),
    MisOptions(tis_level="token", tis_mode="truncate", use_rs=True, rs_level="geometric", rs_lower_bound=0.9, rs_upper_bound=1.1),
    MisOptions(tis_level="token", tis_mode="clip", use_rs=True, rs_level="token", rs_veto_threshold=0.5),
    MisOptions(use_tis=False, use_rs=True, rs_level="sequence", rs_lower_bound=0.5, rs_upper_bound=2.0),
])
def test_weights_and_masks_match_the_per_sample_loop(opts):
    train, rollout, mask, seg, S = _batch(3)
    w, nm, metrics = mis_weights(train, rollout, mask, seg, opts, S)
    ow, om = _oracle(train, rollout, mask, seg, S, opts)
    assert torch.equal(nm, om)
    if opts.use_tis:
        assert torch.allclose(w, ow, atol=1e-6)
    else:
        assert w is None
    assert "mismatch_abs_logprob_diff" in metrics and all(v.shape == train.shape for v in metrics.values())
    assert torch.allclose(metrics["rejected_token_fraction"], mask - om)


def test_batch_normalisation_and_bad_options():
    train, rollout, mask, seg, S = _batch(5)
    w, _, m = mis_weights(train, rollout, mask, seg, MisOptions(tis_mode="clip", tis_batch_normalize=True), S)
    assert (w * mask).sum().item() / mask.sum().item() == pytest.approx(1.0, rel=1e-5)
    w, _, _ = mis_weights(train, rollout, mask, seg, MisOptions(tis_level="sequence", tis_batch_normalize=True), S)
    per = torch.stack([(w * mask)[seg == s].sum() / mask[seg == s].sum().clamp_min(1) for s in range(S) if mask[seg == s].sum() > 0])
    assert per.mean().item() == pytest.approx(1.0, rel=1e-5)
    with pytest.raises(ValueError):
        MisOptions.from_args(SimpleNamespace(tis_level="paragraph"))


def test_plug_in_changes_the_policy_loss_through_the_hook():
    from miles_b200.rl.losses import LossConfig, SegmentReducer, policy_loss

    train, rollout, mask, seg, S = _batch(9)
    adv = torch.randn(train.numel())
    lp = train.clone().requires_grad_(True)
    args = SimpleNamespace(tis_level="token", tis_mode="truncate", tis_upper_bound=1.3, use_rs=True, rs_level="token",
                           rs_lower_bound=0.6, rs_upper_bound=1.6)
    cfg = LossConfig(use_tis=True, custom_tis_fn=mis_function)
    cfg.args = args
    red = SegmentReducer(seg, mask, num_samples=S)
    loss, metrics = policy_loss(cfg, lp, None, old_log_probs=train, advantages=adv, reducer=red, rollout_log_probs=rollout)
    opts = MisOptions.from_args(args)
    w, nm, _ = mis_weights(train, rollout, mask, seg, opts, S)
    # on-policy step: the ratio is one, the per-token loss is -advantage; weights and the rejection mask apply on top
    want = SegmentReducer(seg, mask, num_samples=S).with_mask(nm)(-adv * w)
    assert loss.item() == pytest.approx(want.item(), rel=1e-5, abs=1e-7)
    assert "tis_truncate_fraction" in metrics and "rs_mask_fraction_low" in metrics and "ois" in metrics
