"""Submission pacing (group vs sample back-fill) and the true-on-policy contract report."""
import asyncio

from miles_b200.models import get_config
from miles_b200.rollout.submission import SubmissionPacer
from miles_b200.true_on_policy import check, explain


def test_group_pacing_counts_groups():
    p = SubmissionPacer("group", 4)
    assert p.may_submit(pending_groups=1, group_budget=2) and not p.may_submit(2, 2)


def test_sample_backfill_admits_a_group_once_enough_samples_finished():
    async def run():
        p = SubmissionPacer("sample", group_size=4)
        p.submitted([[0] * 4, [0] * 4])
        assert not p.may_submit(pending_groups=2, group_budget=2)  # 8 in flight, budget 8
        slow = asyncio.ensure_future(asyncio.sleep(10))
        for _ in range(3):
            p.sample_finished()
        assert not p.may_submit(2, 2)  # 5 in flight + 4 > 8
        asyncio.get_event_loop().call_later(0.01, p.sample_finished)
        done, rest = await p.wait({slow})
        assert not done and rest == {slow}  # woken by the sample, not by a group
        assert p.may_submit(2, 2)  # 4 in flight + 4 <= 8
        slow.cancel()
        p.submitted([[0] * 4])
        assert p.may_submit(pending_groups=0, group_budget=1) and p.samples_in_flight == 0  # stale count dropped

    asyncio.run(run())


def test_contract_names_what_breaks_bit_equality():
    class A:
        use_rollout_routing_replay = False
        sglang_quantization = None

    rep = check(A(), get_config("qwen3-30B-A3B"))
    assert {c.key for c in rep.broken} == {"routing", "attention", "batch_invariance"} and not rep.bitwise_expected
    A.use_rollout_routing_replay = True
    assert "routing" in {c.key for c in check(A(), get_config("qwen3-30B-A3B")).satisfied}
    assert "routing" in {c.key for c in check(A(), get_config("qwen3-4B")).satisfied}
    assert "broken: attention" in explain(rep)


def test_rollout_loop_paces_by_sample_and_by_group():
    """The whole loop under both granularities: same batch, same rewards; by sample the pacer's in-flight count returns
    to zero and new groups were admitted while others were still generating."""
    from miles_b200.loop import RLLoop
    from miles_b200.utils.arguments import parse_args

    base = ["--model-preset", "qwen3-tiny", "--rollout-batch-size", "4", "--n-samples-per-prompt", "4", "--rollout-max-response-len", "8",
            "--rollout-max-prompt-len", "16", "--rm-type", "parity", "--lr", "1e-5", "--micro-batch-size", "8", "--colocate",
            "--num-rollout", "1", "--actor-num-gpus-per-node", "1", "--over-sampling-batch-size", "4"]
    outs = {}
    for g in ("group", "sample"):
        loop = RLLoop(parse_args(base + ["--rollout-submission-granularity", g]))
        samples, _ = loop.generate(0)
        assert len(samples) == 16
        outs[g] = sorted((s.index, tuple(s.tokens), s.reward) for s in samples)
        pacer = loop.rollout_fn.state.pacer
        assert pacer.by_sample == (g == "sample") and pacer.samples_in_flight == 0
    assert outs["group"] == outs["sample"]


def test_rollout_logprobs_recomputed_through_the_engines_prefill():
    """--recompute-logprobs-via-prefill: the recorded rollout log-probs are the engine's one-pass scores of the finished
    sequence; in fp32 they equal the ones recorded while decoding and the trainer's."""
    from miles_b200.loop import RLLoop
    from miles_b200.utils.arguments import parse_args

    base = ["--model-preset", "qwen3-tiny", "--rollout-batch-size", "4", "--n-samples-per-prompt", "2", "--rollout-max-response-len", "8",
            "--rollout-max-prompt-len", "16", "--rm-type", "parity", "--lr", "1e-5", "--micro-batch-size", "8", "--colocate",
            "--num-rollout", "1", "--actor-num-gpus-per-node", "1"]
    plain = RLLoop(parse_args(base)).generate(0)[0]
    loop = RLLoop(parse_args(base + ["--recompute-logprobs-via-prefill"]))
    scored = loop.generate(0)[0]
    assert loop.engine.stats.get("scored_tokens", 0) > 0
    for a, b in zip(sorted(plain, key=lambda s: s.index), sorted(scored, key=lambda s: s.index)):
        assert a.tokens == b.tokens and b.metadata["rollout_log_probs_source"] == "prefill_recompute"
        assert len(b.rollout_log_probs) == b.response_length
        assert max(abs(x - y) for x, y in zip(a.rollout_log_probs, b.rollout_log_probs)) < 1e-4
