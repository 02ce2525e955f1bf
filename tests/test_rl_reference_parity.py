"""RL math against the reference's own functions (miles/backends/training_utils/loss_hub/math_utils.py), imported from
an unmodified install of the reference under ``baseline/_ref`` when that install is present. Random inputs, fp32, CPU."""
import os
import sys
import warnings
from argparse import Namespace

import pytest
import torch

_REF = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref")


def _ref_math():
    if not os.path.isdir(os.path.join(_REF, "miles")):
        pytest.skip("the reference is not installed under baseline/_ref")
    if _REF not in sys.path:
        sys.path.append(_REF)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        try:
            import miles.backends.training_utils.loss_hub.math_utils as m
        except Exception as e:  # noqa: BLE001  (a dependency of the reference that this image lacks)
            pytest.skip(f"the reference's math module does not import here: {e!r}")
    return m


@pytest.fixture(autouse=True)
def _eager_reference():
    """The reference decorates some of these functions with torch.compile; run them as plain Python (no C++ toolchain
    for the inductor here, and the test is about the math)."""
    with torch.compiler.set_stance("force_eager"):
        yield


@pytest.mark.parametrize("T,chunk", [(7, 128), (128, 128), (300, 128), (1000, 64)])
def test_gae_matches_reference(T, chunk):
    m = _ref_math()
    from miles_b200.rl.advantages import chunked_gae, vanilla_gae
    g = torch.Generator().manual_seed(T)
    r, v = torch.randn(3, T, generator=g), torch.randn(3, T, generator=g)
    for gamma, lam in ((1.0, 1.0), (0.99, 0.95), (0.9, 0.5)):
        want_a, want_r = m.vanilla_gae(r, v, gamma, lam)
        for fn in (vanilla_gae, lambda *a: chunked_gae(*a, chunk)):
            a, ret = fn(r, v, gamma, lam)
            torch.testing.assert_close(a, want_a, rtol=2e-4, atol=2e-4)
            torch.testing.assert_close(ret, want_r, rtol=2e-4, atol=2e-4)
        ca, cr = m.chunked_gae(r, v, gamma, lam, chunk)
        torch.testing.assert_close(chunked_gae(r, v, gamma, lam, chunk)[0], ca, rtol=2e-4, atol=2e-4)


@pytest.mark.parametrize("kind", ["k1", "k2", "k3", "low_var_kl"])
@pytest.mark.parametrize("with_ratio", [False, True])
def test_approx_kl_matches_reference(kind, with_ratio):
    m = _ref_math()
    from miles_b200.rl.kl import compute_approx_kl
    g = torch.Generator().manual_seed(3)
    lp, base = -torch.rand(500, generator=g) * 5, -torch.rand(500, generator=g) * 5
    lp[:3] = torch.tensor([-30.0, 0.0, -0.5])   # extreme differences reach the clamps of low_var_kl
    base[:3] = torch.tensor([0.0, -30.0, -0.5])
    ir = torch.rand(500, generator=g) * 2 if with_ratio else None
    torch.testing.assert_close(compute_approx_kl(lp, base, kind, ir), m.compute_approx_kl(lp, base, kind, ir), rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("eps_c", [None, 3.0])
def test_clipped_policy_loss_matches_reference(eps_c):
    m = _ref_math()
    from miles_b200.rl.losses import compute_policy_loss
    g = torch.Generator().manual_seed(5)
    kl = torch.randn(2000, generator=g) * 0.5
    adv = torch.randn(2000, generator=g)
    loss, frac = compute_policy_loss(kl, adv, 0.2, 0.28, eps_c)
    want_loss, want_frac = m.compute_policy_loss(kl, adv, 0.2, 0.28, eps_c)
    torch.testing.assert_close(loss, want_loss, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(frac.float(), want_frac.float())


def _samples(seed, n=5):
    g = torch.Generator().manual_seed(seed)
    lens = [int(x) for x in torch.randint(3, 40, (n,), generator=g)]
    new = [-torch.rand(L, generator=g) * 3 for L in lens]
    old = [x + torch.randn(L, generator=g) * 0.2 for x, L in zip(new, lens)]
    masks = [(torch.rand(L, generator=g) > 0.2).float() for L in lens]
    for mk in masks:
        mk[-1] = 1.0
    adv = [torch.randn(L, generator=g) for L in lens]
    return lens, new, old, masks, adv


def _flat(lens, *lists):
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int64)
    return (cu,) + tuple(torch.cat(x) for x in lists)


def test_gspo_sequence_kl_matches_reference():
    m = _ref_math()
    from miles_b200.rl.advantages import seg_ids
    from miles_b200.rl.losses import SegmentReducer
    lens, new, old, masks, _ = _samples(11)
    want = m.compute_gspo_kl(new, old, new, masks)          # per-token tensor: each token carries its sequence's KL
    cu, fn, fo, fm = _flat(lens, new, old, masks)
    red = SegmentReducer(seg_ids(cu), fm, per_token=False)
    got = red.seq_mean(fo - fn)[red.seg]
    torch.testing.assert_close(got, want, rtol=1e-5, atol=1e-6)


def test_opsm_mask_matches_reference():
    m = _ref_math()
    from miles_b200.rl.advantages import seg_ids
    from miles_b200.rl.losses import LossConfig, SegmentReducer, policy_loss
    lens, new, old, masks, adv = _samples(13, n=8)
    delta = 0.01
    want_mask, want_clipfrac = m.compute_opsm_mask(Namespace(opsm_delta=delta), new, old, adv, masks)
    cu, fn, fo, fm, fa = _flat(lens, new, old, masks, adv)
    red = SegmentReducer(seg_ids(cu), fm, per_token=False)
    seq_kl = red.seq_mean(fo - fn)
    got_mask = 1.0 - ((fa < 0) & (seq_kl[red.seg] > delta)).float()
    torch.testing.assert_close(got_mask, want_mask.float())
    cfg = LossConfig(use_opsm=True, opsm_delta=delta)
    _, metrics = policy_loss(cfg, fn.clone().requires_grad_(True), None, old_log_probs=fo, advantages=fa, reducer=red)
    assert float(want_clipfrac) > 0.0, "the case must drop something"
    torch.testing.assert_close(metrics["opsm_clipfrac"], want_clipfrac, rtol=1e-5, atol=1e-6)


def test_group_returns_and_reinforce_match_reference():
    m = _ref_math()
    from miles_b200.rl.advantages import compute_advantages_and_returns
    lens, new, old, masks, _ = _samples(17, n=6)
    rewards = torch.randn(6)
    kl = [torch.zeros(L) for L in lens]
    cu, fm, fn, fo = _flat(lens, masks, new, old)
    want = torch.cat(m.get_grpo_returns(rewards, kl))
    adv, ret, _ = compute_advantages_and_returns(advantage_estimator="grpo", rewards=rewards, cu=cu, loss_mask=fm)
    torch.testing.assert_close(adv, want)
    torch.testing.assert_close(ret, want)
    # REINFORCE++-baseline with a KL penalty: A_t = r - kl_coef * KL_t
    kls = [(n_ - o_) for n_, o_ in zip(new, old)]
    want = torch.cat(m.get_reinforce_plus_plus_baseline_advantages(rewards, kls, masks, 0.05))
    adv, _, _ = compute_advantages_and_returns(advantage_estimator="reinforce_plus_plus_baseline", rewards=rewards, cu=cu,
                                               loss_mask=fm, log_probs=fn, ref_log_probs=fo, kl_coef=0.05, kl_loss_type="k1")
    torch.testing.assert_close(adv, want, rtol=1e-5, atol=1e-6)
    # REINFORCE++: discounted return of -kl_coef*KL_t with the reward on the last trainable token. The reference reads
    # the context-parallel size from its global parallel state: give it a single-rank stand-in.
    import miles.backends.training_utils.parallel as ref_parallel
    from types import SimpleNamespace
    ref_parallel.set_parallel_state(SimpleNamespace(cp=SimpleNamespace(size=1, rank=0)))
    want = torch.cat(m.get_reinforce_plus_plus_returns(rewards, kls, masks, lens, [L + 4 for L in lens], 0.05, 0.97))
    adv, _, _ = compute_advantages_and_returns(advantage_estimator="reinforce_plus_plus", rewards=rewards, cu=cu, loss_mask=fm,
                                               log_probs=fn, ref_log_probs=fo, kl_coef=0.05, kl_loss_type="k1", gamma=0.97)
    torch.testing.assert_close(adv * fm, want * fm, rtol=1e-4, atol=1e-5)
