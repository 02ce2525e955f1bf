"""RL mathematics on CPU: GAE (chunked vs loop), KL estimators, reward normalisation, advantages, losses."""

import pytest
import torch

from miles_b200.rl import (SegmentReducer, chunked_gae, compute_advantages_and_returns, compute_approx_kl,
                           normalize_group_rewards, policy_loss, sft_loss, value_loss, vanilla_gae, whiten)
from miles_b200.rl.advantages import gae_flat, last_trainable_index, seg_ids
from miles_b200.rl.losses import LossConfig, compute_policy_loss


@pytest.mark.parametrize("B,T", [(1, 1), (3, 127), (4, 128), (2, 129), (5, 1000)])
@pytest.mark.parametrize("gamma,lam", [(1.0, 1.0), (0.99, 0.95), (0.9, 0.5)])
def test_chunked_gae_matches_loop(B, T, gamma, lam):
    torch.manual_seed(T)
    r, v = torch.randn(B, T, dtype=torch.float64), torch.randn(B, T, dtype=torch.float64)
    a0, ret0 = vanilla_gae(r, v, gamma, lam)
    a1, ret1 = chunked_gae(r, v, gamma, lam)
    assert torch.allclose(a0.float(), a1.float(), atol=1e-5, rtol=1e-5)
    assert torch.allclose(ret0.float(), ret1.float(), atol=1e-5, rtol=1e-5)


def test_gae_flat_skips_masked_tokens():
    torch.manual_seed(0)
    cu = torch.tensor([0, 5, 12])
    mask = torch.tensor([1, 1, 0, 1, 1, 0, 1, 1, 1, 0, 0, 1.0])
    r, v = torch.randn(12), torch.randn(12)
    adv, ret = gae_flat(r, v, mask, cu, 0.99, 0.9)
    assert torch.all(adv[mask == 0] == 0)
    # equals GAE on the compacted sequences
    for a, b in ((0, 5), (5, 12)):
        m = mask[a:b].bool()
        ea, _ = vanilla_gae(r[a:b][m][None], v[a:b][m][None], 0.99, 0.9)
        assert torch.allclose(adv[a:b][m], ea[0], atol=1e-5)


def test_kl_estimators():
    lp, base = torch.tensor([-1.0, -2.0, -0.5]), torch.tensor([-1.5, -1.0, -0.5])
    d = lp - base
    assert torch.allclose(compute_approx_kl(lp, base, "k1"), d)
    assert torch.allclose(compute_approx_kl(lp, base, "k2"), d * d / 2)
    assert torch.allclose(compute_approx_kl(lp, base, "k3"), torch.exp(-d) - 1 + d)
    big = compute_approx_kl(torch.tensor([-100.0]), torch.tensor([0.0]), "low_var_kl")
    assert big.item() == 10.0
    w = torch.tensor([0.5, 2.0, 1.0])
    assert torch.allclose(compute_approx_kl(lp, base, "k2", w), w * d * d / 2)
    with pytest.raises(ValueError):
        compute_approx_kl(lp, base, "nope")


def test_group_reward_normalisation():
    r = [1.0, 0.0, 1.0, 1.0, 0.0, 0.0, 0.0, 0.0]
    g = [0, 0, 0, 0, 1, 1, 1, 1]
    out = normalize_group_rewards(r, g, advantage_estimator="grpo")
    v = torch.tensor(r[:4])
    exp = (v - v.mean()) / (v.std() + 1e-6)
    assert torch.allclose(torch.tensor(out[:4]), exp, atol=1e-6)
    assert out[4:] == [0.0, 0.0, 0.0, 0.0]  # zero std: centred only
    # multi-sample rollouts count once
    out2 = normalize_group_rewards([1.0, 1.0, 0.0], [0, 0, 0], [7, 7, 8], advantage_estimator="grpo")
    v = torch.tensor([1.0, 0.0])
    e2 = (v - v.mean()) / (v.std() + 1e-6)
    assert abs(out2[0] - e2[0].item()) < 1e-6 and out2[0] == out2[1] and abs(out2[2] - e2[1].item()) < 1e-6
    assert normalize_group_rewards(r, g, advantage_estimator="ppo") == r
    assert normalize_group_rewards(r, g, advantage_estimator="grpo", std_normalization=False)[:4] == [0.25, -0.75, 0.25, 0.25]


def test_advantage_estimators():
    cu = torch.tensor([0, 3, 7])
    mask = torch.tensor([1, 1, 1, 1, 0, 1, 0.0])
    rewards = torch.tensor([2.0, -1.0])
    adv, ret, kl = compute_advantages_and_returns(advantage_estimator="grpo", rewards=rewards, cu=cu, loss_mask=mask)
    assert adv.tolist() == [2, 2, 2, -1, -1, -1, -1] and kl.abs().sum() == 0
    assert last_trainable_index(mask, cu).tolist() == [2, 5]
    lp, ref = torch.randn(7), torch.randn(7)
    adv, ret, kl = compute_advantages_and_returns(advantage_estimator="reinforce_plus_plus", rewards=rewards, cu=cu, loss_mask=mask,
                                                  log_probs=lp, ref_log_probs=ref, kl_coef=0.1, gamma=0.9)
    tok_r = -0.1 * (lp - ref)
    tok_r[2] += 2.0
    tok_r[5] += -1.0
    exp = torch.zeros(7)
    for a, b in ((0, 3), (3, 7)):
        run = 0.0
        for t in reversed(range(a, b)):
            run = tok_r[t] + 0.9 * run
            exp[t] = run
    assert torch.allclose(adv, exp, atol=1e-5)
    adv, _, _ = compute_advantages_and_returns(advantage_estimator="reinforce_plus_plus_baseline", rewards=rewards, cu=cu,
                                               loss_mask=mask, log_probs=lp, ref_log_probs=ref, kl_coef=0.1)
    assert torch.allclose(adv, rewards[seg_ids(cu)] - 0.1 * (lp - ref))
    vals = torch.randn(7)
    adv, ret, _ = compute_advantages_and_returns(advantage_estimator="ppo", rewards=rewards, cu=cu, loss_mask=mask, values=vals,
                                                 log_probs=lp, ref_log_probs=ref, kl_coef=0.0, gamma=1.0, lambd=1.0)
    # gamma = lambda = 1: advantage = (sum of future rewards) - V_t on trainable tokens
    assert abs(adv[0].item() - (2.0 - vals[0].item())) < 1e-5
    assert adv[4].item() == 0 and abs(adv[3].item() - (-1.0 - vals[3].item())) < 1e-5


def test_whiten():
    x = torch.tensor([1.0, 2.0, 3.0, 100.0])
    m = torch.tensor([1.0, 1.0, 1.0, 0.0])
    w = whiten(x, m)
    assert abs(w[:3].mean().item()) < 1e-6
    assert abs(w[:3].std(unbiased=True).item() - 1.0) < 1e-3


def _reducer(mask, cu, per_token=False, denoms=None):
    return SegmentReducer(seg_ids(cu), mask, denoms, per_token)


def test_policy_loss_on_policy_is_minus_mean_advantage():
    cu = torch.tensor([0, 4, 6])
    mask = torch.tensor([1, 1, 0, 1, 1, 1.0])
    lp = torch.randn(6, requires_grad=True)
    adv = torch.tensor([1.0, 1.0, 1.0, 1.0, -2.0, -2.0])
    cfg = LossConfig()
    loss, m = policy_loss(cfg, lp, None, old_log_probs=lp.detach(), advantages=adv, reducer=_reducer(mask, cu))
    assert abs(loss.item() - (-(1.0) + 2.0)) < 1e-6  # per-sample mean of -A summed over samples
    assert m["ppo_kl"].abs().item() < 1e-9 and m["pg_clipfrac"].item() == 0
    loss.backward()
    # gradient of -ratio*A at ratio 1 is -A * mask / denominators
    exp = -adv * mask / torch.tensor([3, 3, 3, 3, 2, 2.0])
    assert torch.allclose(lp.grad, exp, atol=1e-6)


def test_policy_loss_clipping_dual_clip_gspo_opsm_tis():
    cu = torch.tensor([0, 3, 6])
    mask = torch.ones(6)
    old = torch.zeros(6)
    lp = torch.tensor([0.5, -0.5, 0.0, 0.5, -0.5, 0.0])
    adv = torch.tensor([1.0, 1.0, 1.0, -1.0, -1.0, -1.0])
    pg, clip = compute_policy_loss(old - lp, adv, 0.2, 0.28)
    r = torch.exp(lp)
    assert torch.allclose(pg[0], -torch.tensor(1.28)) and clip[0] == 1  # ratio 1.65 clipped at 1.28 for A>0
    assert torch.allclose(pg[1], -r[1]) and clip[1] == 0  # ratio below 1-eps with A>0: unclipped is larger
    assert torch.allclose(pg[4], torch.tensor(0.8)) and clip[4] == 1
    pg3, _ = compute_policy_loss(torch.tensor([-3.0]), torch.tensor([-1.0]), 0.2, 0.2, 3.0)
    assert abs(pg3.item() - 3.0) < 1e-6  # dual clip bounds the loss at c*|A|
    cfg = LossConfig(advantage_estimator="gspo")
    lpg = lp.clone().requires_grad_(True)
    loss, m = policy_loss(cfg, lpg, None, old_log_probs=old, advantages=adv, reducer=_reducer(mask, cu))
    assert abs(m["ppo_kl"].item() - 0.0) < 1e-6  # sequence means of (old - new) are zero here
    cfg = LossConfig(use_opsm=True, opsm_delta=0.1)
    lp2 = torch.tensor([0.0, 0.0, 0.0, -1.0, -1.0, -1.0])
    loss, m = policy_loss(cfg, lp2, None, old_log_probs=old, advantages=adv, reducer=_reducer(mask, cu))
    assert abs(m["opsm_clipfrac"].item() - 1.0) < 1e-6  # second sequence (A<0, seq KL 1 > delta) is dropped
    cfg = LossConfig(use_tis=True, tis_clip=2.0, tis_clip_low=0.5)
    roll = torch.tensor([0.0, -1.0, 1.0, 0.0, 0.0, 0.0])
    loss, m = policy_loss(cfg, old.clone(), None, old_log_probs=old, advantages=adv, reducer=_reducer(mask, cu), rollout_log_probs=roll)
    assert abs(m["tis_clipfrac"].item() - (2 / 3)) < 1e-6
    cfg.tis_mode = "icepop"
    loss2, _ = policy_loss(cfg, old.clone(), None, old_log_probs=old, advantages=adv, reducer=_reducer(mask, cu), rollout_log_probs=roll)
    assert abs(loss2.item() - (-(1 / 3) + 1.0)) < 1e-6


def test_kl_loss_entropy_and_metrics():
    cu = torch.tensor([0, 4])
    mask = torch.ones(4)
    lp = torch.tensor([-1.0, -2.0, -0.5, -1.5], requires_grad=True)
    ref = torch.tensor([-1.2, -1.5, -0.5, -1.0])
    ent = torch.tensor([1.0, 2.0, 3.0, 4.0], requires_grad=True)
    cfg = LossConfig(use_kl_loss=True, kl_loss_coef=0.5, kl_loss_type="k2", entropy_coef=0.1)
    loss, m = policy_loss(cfg, lp, ent, old_log_probs=lp.detach(), advantages=torch.zeros(4), reducer=_reducer(mask, cu),
                          ref_log_probs=ref, rollout_log_probs=lp.detach() + 0.01)
    kl = ((lp.detach() - ref) ** 2 / 2).mean()
    assert abs(m["kl_loss"].item() - kl.item()) < 1e-6
    assert abs(loss.item() - (0.5 * kl.item() - 0.1 * 2.5)) < 1e-6
    assert abs(m["train_rollout_logprob_abs_diff"].item() - 0.01) < 1e-6
    assert m["ess_ratio"].item() == pytest.approx(1.0)


def test_value_and_sft_loss_and_denominators():
    cu = torch.tensor([0, 2, 4])
    mask = torch.ones(4)
    red = _reducer(mask, cu, denoms=torch.tensor([4.0, 4.0]))  # both samples belong to one 4-token rollout
    v = torch.tensor([1.0, 2.0, 3.0, 4.0])
    loss, m = value_loss(LossConfig(value_clip=0.5), v, old_values=v - 1.0, returns=torch.zeros(4), reducer=red)
    assert abs(loss.item() - (1 + 4 + 9 + 16) / 4) < 1e-6 and m["value_clipfrac"].item() == 1.0
    lp = torch.tensor([-1.0, -1.0, -3.0, -3.0])
    assert abs(sft_loss(LossConfig(), lp, reducer=_reducer(mask, cu))[0].item() - 4.0) < 1e-6
    assert abs(sft_loss(LossConfig(), lp, reducer=_reducer(mask, cu, per_token=True))[0].item() - 8.0) < 1e-6
