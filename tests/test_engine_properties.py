"""Property test of the engine's page accounting and of what caching may change: random mixes of prompts with shared
starts, generation lengths, cache flushes, weight-version bumps and prefix hand-overs between two engines. Whatever the
sequence, (a) no page leaks: free + cached pages add up to the pool once nothing runs, (b) tokens equal those of an engine
without any cache, (c) a hand-over never imports across weight versions."""
import pytest
import torch

hypothesis = pytest.importorskip("hypothesis")
from hypothesis import HealthCheck, given, settings  # noqa: E402
from hypothesis import strategies as st  # noqa: E402

from miles_b200.engine import Engine, SamplingParams  # noqa: E402
from miles_b200.models import ParamStore, build_model, get_config  # noqa: E402

CFG = get_config("qwen3-tiny")
STORE = ParamStore(CFG, "cpu", torch.float32, seed=11)
MODEL = build_model(CFG, STORE)
BASES = [torch.randint(0, CFG.vocab_size, (40,), generator=torch.Generator().manual_seed(s)).tolist() for s in range(3)]

prompt = st.tuples(st.integers(0, 2), st.integers(3, 40), st.lists(st.integers(0, CFG.vocab_size - 1), max_size=6))
op = st.one_of(
    st.tuples(st.just("gen"), st.lists(st.tuples(prompt, st.integers(1, 9)), min_size=1, max_size=4)),
    st.tuples(st.just("flush"), st.none()),
    st.tuples(st.just("handover"), prompt),
    st.tuples(st.just("bump"), st.none()),
)


def _ids(p):
    base, n, tail = p
    return BASES[base][:n] + list(tail)


def _check_pages(e):
    assert not e.running and not e.waiting
    cached = e.prefix.num_pages if e.prefix is not None else 0
    assert e.pool.num_free + cached == e.num_pages - 1, (e.pool.num_free, cached, e.num_pages)


@settings(max_examples=60, deadline=None, suppress_health_check=[HealthCheck.too_slow, HealthCheck.data_too_large])
@given(st.lists(op, min_size=1, max_size=6), st.integers(10, 40))
def test_random_operation_sequences_keep_pages_and_outputs(ops, num_pages):
    plain = Engine(MODEL, max_running=4, page_size=8, max_seq_len=64)
    a = Engine(MODEL, max_running=4, page_size=8, max_seq_len=64, num_pages=num_pages, prefix_cache=True)
    b = Engine(MODEL, max_running=4, page_size=8, max_seq_len=64, num_pages=num_pages, prefix_cache=True)
    seed = 0
    for kind, arg in ops:
        if kind == "gen":
            prompts = [_ids(p) for p, _ in arg]
            sps = []
            for _, n in arg:
                seed += 1
                sps.append(SamplingParams(max_new_tokens=n, sampling_seed=seed, ignore_eos=True))
            want = plain.generate(prompts, sps)
            for e in (a, b):
                got = e.generate(prompts, sps)
                assert [g["output_ids"] for g in got] == [w["output_ids"] for w in want]
                _check_pages(e)
        elif kind == "flush":
            assert a.flush_cache() and a.prefix.num_pages == 0
            _check_pages(a)
        elif kind == "bump":
            b.update_weight_version()          # b now serves "newer" weights than a
            b.flush_cache()
        else:
            ids = _ids(arg)
            blob = a.export_prefix(ids)
            before = b.prefix.num_pages
            got = b.import_prefix(blob)
            if blob is None or a.weight_version != b.weight_version:
                assert got == 0 and b.prefix.num_pages == before
            else:
                assert got % 8 == 0 and got <= len(blob["tokens"])
            _check_pages(b)
    for e in (plain, a, b):
        _check_pages(e) if e.prefix is not None else None
