"""Audit trail: witness ring and allocator, event log with a resumable sequence, analyzer rules, and the whole thing
inside the training loop (exactly-once training proven from the table's own read-back)."""
import torch

from miles_b200.utils.audit import (EventLogger, Witness, WitnessAllocator, analyze, ev_engine_checksum, ev_train_step,
                                     ev_weight_checksum, ev_witness_allocate, ev_witness_snapshot, read_events)


def test_allocator_ring_reuses_slots_and_reports_stale_ids():
    a = WitnessAllocator(4)
    w0, s0 = a.allocate(0, [10, 11, 12])
    assert w0 == [0, 1, 2] and s0 == []
    assert a.allocate(0, [11, 12]) == ([1, 2], [])          # a retried rollout gets its slots again
    w1, s1 = a.allocate(1, [5, 6, 7])
    assert w1 == [3, 0, 1] and s1 == [0, 1]                 # the ring wrapped over rollout 0's first two slots
    b = WitnessAllocator(4)
    b.load_state_dict(a.state_dict())
    assert b.allocate(1, [6]) == ([0], []) and b.next == a.next


def test_witness_counts_commit_discard_and_stale_reset():
    w = Witness(4)
    ids, _ = w.allocate(0, [0, 1, 2])
    w.touch(ids)
    w.discard()
    assert w.counts(ids) == {0: 0, 1: 0, 2: 0}
    w.touch(ids)
    w.touch(ids[:1])
    w.commit()
    assert w.counts(ids) == {0: 2, 1: 1, 2: 1}
    ids2, stale = w.allocate(1, [7, 8])
    assert ids2 == [3, 0] and stale == [0] and w.counts([0]) == {0: 0}   # the reused slot starts from zero
    w2 = Witness(4)
    w2.load_state_dict(w.state_dict())
    assert torch.equal(w2.table, w.table)


def test_event_log_round_trip_and_sequence_survives_resume(tmp_path):
    log = EventLogger(str(tmp_path), "actor", 0)
    log.log(ev_weight_checksum(1, 1, "1.0e+00"))
    log.log("cell_state", cell=0, state="healthy")
    sd = log.state_dict()
    again = EventLogger(str(tmp_path), "actor", 0)
    again.load_state_dict(sd)
    again.log(ev_weight_checksum(2, 2, "2.0e+00"))
    evs = read_events(str(tmp_path))
    assert [e["seq"] for e in evs] == [0, 1, 2] and evs[1]["state"] == "healthy" and all(e["role"] == "actor" for e in evs)


def _ident(rank):
    return {"host": "h", "pid": 100 + rank, "role": "actor", "rank": rank, "ts": 0.0}


def test_rules_find_each_kind_of_inconsistency():
    ok = [dict(ev_weight_checksum(1, 1, "a"), **_ident(0)), dict(ev_weight_checksum(1, 1, "a"), **_ident(1)),
          dict(ev_engine_checksum("e0", 1, "a"), **_ident(0))]
    assert analyze(ok) == []
    bad = ok + [dict(ev_weight_checksum(2, 2, "b"), **_ident(0)), dict(ev_weight_checksum(2, 2, "c"), **_ident(1)),
                dict(ev_engine_checksum("e1", 1, "zzz"), **_ident(0))]
    probs = analyze(bad)
    assert any("disagree" in p and "step 2" in p for p in probs) and any("engine e1" in p for p in probs)
    assert analyze(bad, rules=["engine_checksum_consistency"]) == [p for p in probs if "engine e1" in p]
    # witness: sample 1 trained twice, sample 2 never, sample 3 only in a discarded step (fine: reads 0)
    w = [dict(ev_witness_allocate(0, [0, 1, 2, 3], [0, 1, 2, 3], []), **_ident(0)),
         dict(ev_train_step(0, 1, 2, "normal", [0, 1]), **_ident(0)),
         dict(ev_train_step(0, 1, 1, "discarded", [3]), **_ident(0)),
         dict(ev_train_step(0, 2, 1, "normal", [2]), **_ident(0)),
         dict(ev_witness_snapshot(0, 2, {0: 1, 1: 2, 2: 0, 3: 0}), **_ident(0))]
    probs = analyze(w, rules=["witness_exactly_once"])
    assert len(probs) == 2 and any("sample 1" in p and "2 times" in p for p in probs) and any("sample 2" in p and "0 times" in p for p in probs)


def test_loop_proves_exactly_once_training(tmp_path):
    from miles_b200.loop import RLLoop
    from miles_b200.utils.arguments import parse_args

    args = parse_args(["--model-preset", "qwen3-tiny", "--rollout-batch-size", "4", "--n-samples-per-prompt", "2", "--rollout-max-response-len", "8",
                       "--rollout-max-prompt-len", "16", "--rm-type", "parity", "--lr", "1e-5", "--micro-batch-size", "4", "--colocate",
                       "--num-rollout", "2", "--actor-num-gpus-per-node", "1", "--num-steps-per-rollout", "2", "--enable-witness",
                       "--enable-event-analyzer", "--save-debug-event-data", str(tmp_path / "events")])
    loop = RLLoop(args)
    loop.run()          # the analyzer runs at the end of run() and asserts on any violation
    evs = read_events(str(tmp_path / "events"))
    kinds = [e["kind"] for e in evs]
    assert kinds.count("witness_allocate") == 2 and kinds.count("train_step") == 4 and kinds.count("witness") == 4
    snap = [e for e in evs if e["kind"] == "witness"]
    assert all(set(e["counts"].values()) == {1} for e in snap)
    assert sorted(int(k) for e in snap for k in e["counts"]) == list(range(16))   # 2 rollouts x 8 samples, each slot once
    # tamper: count one sample twice -> the analyzer notices
    loop.actor.witness.touch([3])
    loop.actor.witness.commit()
    from miles_b200.utils.audit import ev_witness_snapshot as snapshot
    loop.actor.events.log(snapshot(0, 99, loop.actor.witness.counts([3])))
    assert any("2 times" in p for p in analyze(read_events(str(tmp_path / "events"))))


def test_witness_and_event_sequence_survive_a_checkpoint(tmp_path):
    from miles_b200.loop import RLLoop
    from miles_b200.utils.arguments import parse_args

    base = ["--model-preset", "qwen3-tiny", "--rollout-batch-size", "4", "--n-samples-per-prompt", "2", "--rollout-max-response-len", "8",
            "--rollout-max-prompt-len", "16", "--rm-type", "parity", "--lr", "1e-5", "--micro-batch-size", "8", "--colocate",
            "--actor-num-gpus-per-node", "1", "--enable-witness", "--save-debug-event-data", str(tmp_path / "events"),
            "--save", str(tmp_path / "ckpt"), "--save-interval", "1"]
    for fmt in ("torch_dist", "torch"):
        a = RLLoop(parse_args(base + ["--num-rollout", "1", "--ckpt-format", fmt]))
        a.run()
        b = RLLoop(parse_args(base + ["--num-rollout", "2", "--ckpt-format", fmt, "--load", str(tmp_path / "ckpt")]))
        assert b.start_rollout_id == 1
        assert torch.equal(b.actor.witness.table, a.actor.witness.table) and b.actor.witness.allocator.next == 8
        assert b.actor.events.seq == a.actor.events.seq > 0
