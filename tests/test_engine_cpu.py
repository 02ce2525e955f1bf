"""Rollout engine control flow on CPU (PyTorch op backend): continuous batching, stop conditions, abort,
pause modes, retraction under page pressure, weight versions, async client routing."""
import asyncio

import pytest
import torch

from miles_b200.engine import Engine, SamplingParams
from miles_b200.engine.client import EngineClient, decode_routed_experts
from miles_b200.models import ParamStore, build_model, get_config


def _engine(name="qwen3-tiny", **kw):
    cfg = get_config(name)
    st = ParamStore(cfg, "cpu", torch.float32, seed=11)
    m = build_model(cfg, st)
    kw.setdefault("max_running", 4)
    kw.setdefault("page_size", 8)
    kw.setdefault("max_seq_len", 128)
    return cfg, m, Engine(m, **kw)


def _prompts(cfg, lens, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in lens]


def test_continuous_batching_more_requests_than_slots_and_parity():
    cfg, m, eng = _engine()
    prompts = _prompts(cfg, [5, 17, 9, 30, 3, 12, 8])
    sps = [SamplingParams(max_new_tokens=n, sampling_seed=i) for i, n in enumerate([4, 9, 1, 6, 12, 3, 7])]
    res = eng.generate(prompts, sps)
    assert [len(r["output_ids"]) for r in res] == [4, 9, 1, 6, 12, 3, 7]
    assert all(r["meta_info"]["finish_reason"]["type"] == "length" for r in res)
    assert eng.pool.num_free == eng.num_pages - 1 and not eng.running
    for p, r in zip(prompts, res):
        ids = p + r["output_ids"]
        tok, pos, cu = torch.tensor(ids), torch.arange(len(ids)), torch.tensor([0, len(ids)])
        lp, _ = m.forward_logprobs(tok, pos, cu, torch.arange(len(p) - 1, len(ids) - 1), tok[len(p):], 1.0)
        elp = torch.tensor([x[0] for x in r["meta_info"]["output_token_logprobs"]])
        assert torch.allclose(lp, elp, atol=1e-4)


def test_sampling_is_seed_deterministic_and_greedy():
    cfg, m, eng = _engine()
    p = _prompts(cfg, [10])
    a = eng.generate(p, SamplingParams(max_new_tokens=8, sampling_seed=5))[0]["output_ids"]
    b = eng.generate(p, SamplingParams(max_new_tokens=8, sampling_seed=5))[0]["output_ids"]
    c = eng.generate(p, SamplingParams(max_new_tokens=8, sampling_seed=6))[0]["output_ids"]
    assert a == b and a != c
    g1 = eng.generate(p, SamplingParams(max_new_tokens=5, temperature=0.0))[0]
    ids = p[0] + g1["output_ids"]
    tok = torch.tensor(ids)
    h = m.forward_hidden(tok, torch.arange(len(ids)), torch.tensor([0, len(ids)]))
    assert m.logits(h[len(p[0]) - 1:-1]).argmax(-1).tolist() == g1["output_ids"]


def test_stop_tokens_and_forced_length():
    cfg, m, eng = _engine()
    p = _prompts(cfg, [6])
    full = eng.generate(p, SamplingParams(max_new_tokens=20, sampling_seed=1))[0]["output_ids"]
    stop = full[7]
    first = full.index(stop)
    r = eng.generate(p, SamplingParams(max_new_tokens=20, sampling_seed=1, stop_token_ids=(stop,)))[0]
    assert r["output_ids"] == full[:first + 1] and r["meta_info"]["finish_reason"]["type"] == "stop"
    r = eng.generate(p, SamplingParams(max_new_tokens=20, sampling_seed=1, stop_token_ids=(stop,), forced_length=11, ignore_eos=True))[0]
    assert len(r["output_ids"]) == 11


def test_abort_pause_modes_and_weight_versions():
    cfg, m, eng = _engine()
    prompts = _prompts(cfg, [8, 8, 8])
    rids = [eng.add_request(p, SamplingParams(max_new_tokens=30, sampling_seed=i)) for i, p in enumerate(prompts)]
    for _ in range(5):
        eng.step()
    assert eng.abort_request(rids[0]) == 1
    eng.pause_generation("in_place")
    assert eng.step() == [] and len(eng.running) == 2
    eng.update_weight_version(3)
    eng.continue_generation()
    for _ in range(3):
        eng.step()
    eng.pause_generation("retract")
    assert not eng.running and len(eng.waiting) == 2 and eng.flush_cache()
    eng.update_weight_version(4)
    eng.continue_generation()
    while eng.has_work():
        eng.step()
    done = {r.rid: r for r in eng.pop_finished()}
    assert done[rids[0]].finish_reason == "abort"
    for rid in rids[1:]:
        assert len(done[rid].output_ids) == 30
        assert done[rid].weight_versions == [0, 3, 4]  # mixed versions are recorded per sample
    eng.pause_generation("abort")
    eng.continue_generation()


def test_retraction_when_pages_run_out():
    cfg, m, eng = _engine(num_pages=9, page_size=8, max_running=4)
    prompts = _prompts(cfg, [14, 14, 14])
    res = eng.generate(prompts, SamplingParams(max_new_tokens=24, sampling_seed=2))
    assert all(len(r["output_ids"]) == 24 for r in res)
    assert eng.stats["retracted"] > 0 and eng.pool.num_free == 8
    solo = [Engine(m, max_running=1, page_size=8, max_seq_len=128).generate([p], SamplingParams(max_new_tokens=24, sampling_seed=2))[0]
            for p in prompts]
    # a retracted request is re-prefilled with its generated tokens and continues identically
    assert [r["output_ids"] for r in res] == [r["output_ids"] for r in solo]


def test_release_and_resume_memory():
    cfg, m, eng = _engine()
    p = _prompts(cfg, [7])
    a = eng.generate(p, SamplingParams(max_new_tokens=4, sampling_seed=1))[0]["output_ids"]
    eng.release_memory_occupation(("kv_cache", "cuda_graph"))
    assert eng.kv_cache is None and eng.step() == []
    eng.resume_memory_occupation(("kv_cache",))
    assert eng.generate(p, SamplingParams(max_new_tokens=4, sampling_seed=1))[0]["output_ids"] == a


def test_async_client_routes_to_least_loaded_engine_and_returns_routing():
    cfg = get_config("qwen3-tiny-moe")
    st = ParamStore(cfg, "cpu", torch.float32, seed=3)
    m = build_model(cfg, st)
    engines = [Engine(m, max_running=2, page_size=8, max_seq_len=64) for _ in range(2)]
    client = EngineClient(engines)
    prompts = _prompts(cfg, [6, 9, 4, 11])

    async def run():
        payloads = [{"input_ids": p, "sampling_params": {"max_new_tokens": 5, "sampling_seed": i}, "return_routed_experts": True}
                    for i, p in enumerate(prompts)]
        return await asyncio.gather(*[client.generate(pl) for pl in payloads])

    outs = asyncio.run(run())
    assert all(len(o["output_ids"]) == 5 for o in outs)
    assert engines[0].stats["prefill_tokens"] > 0 and engines[1].stats["prefill_tokens"] > 0
    re = decode_routed_experts(outs[1]["meta_info"])
    assert re.shape == (9 + 5 - 1, 2, cfg.moe_top_k) and re.min() >= 0 and re.max() < cfg.num_experts


def test_overlapped_decode_matches_step_by_step_and_handles_unforeseen_stops():
    """One decode step in flight while the host reads the previous one: same tokens as the strictly sequential
    engine, also when a stop token ends a request after the next step was already launched."""
    cfg, m, seq = _engine(overlap_decode=False)
    _, _, ovl = _engine(overlap_decode=True)
    prompts = _prompts(cfg, [9, 21, 5, 14], seed=4)
    base = seq.generate(prompts, SamplingParams(max_new_tokens=20, sampling_seed=5))
    # pick a token that some request produces mid-way and make it a stop token
    stop = base[1]["output_ids"][7]
    sp = SamplingParams(max_new_tokens=20, sampling_seed=5, stop_token_ids=[stop])
    steps0 = seq.stats["decode_steps"]
    a = seq.generate(prompts, sp)
    b = ovl.generate(prompts, sp)
    assert [r["output_ids"] for r in a] == [r["output_ids"] for r in b]
    assert [r["meta_info"]["finish_reason"]["type"] for r in a] == [r["meta_info"]["finish_reason"]["type"] for r in b]
    assert any(r["meta_info"]["finish_reason"]["type"] == "stop" for r in b)
    assert ovl._pending is None and not ovl.running and ovl.pool.num_free == ovl.num_pages - 1
    assert ovl.stats["decode_steps"] >= seq.stats["decode_steps"] - steps0  # speculated steps whose rows were dropped count too


def test_remote_client_balances_and_fans_out():
    from miles_b200.engine.remote import RemoteEngineClient

    calls = []
    gate = asyncio.Event()

    async def transport(method, url, payload):
        calls.append((method, url))
        if url.endswith("/generate"):
            await gate.wait()
            return 200, {"output_ids": [1], "meta_info": {"finish_reason": {"type": "stop"}}}
        if url.endswith("/get_weight_version"):
            return 200, {"weight_version": 3}
        if url.endswith("/health_generate"):
            if "e1" in url:
                raise OSError("down")
            return 200, {"status": "ok"}
        return 200, {"success": True}

    async def main():
        c = RemoteEngineClient(["http://e0/", "http://e1"], transport=transport, max_retries=0)
        tasks = [asyncio.ensure_future(c.generate({"input_ids": [1]})) for _ in range(4)]
        await asyncio.sleep(0.01)
        assert c.inflight == {"http://e0": 2, "http://e1": 2}  # least in flight
        same = [c._pick("session-a") for _ in range(3)]
        assert len(set(same)) == 1  # a session sticks to its engine
        gate.set()
        outs = await asyncio.gather(*tasks)
        assert all(o["output_ids"] == [1] for o in outs) and c.inflight == {"http://e0": 0, "http://e1": 0}
        await c.pause_generation("abort")
        await c.continue_generation()
        assert await c.weight_versions() == [3, 3]
        assert await c.health() == {"http://e0": True, "http://e1": False}
        return c

    asyncio.run(main())
    assert sum(u.endswith("/pause_generation") for _, u in calls) == 2


def _logprob_parity(m, prompts, res, atol=1e-4):
    for p, r in zip(prompts, res):
        ids = p + r["output_ids"]
        tok, pos, cu = torch.tensor(ids), torch.arange(len(ids)), torch.tensor([0, len(ids)])
        lp, _ = m.forward_logprobs(tok, pos, cu, torch.arange(len(p) - 1, len(ids) - 1), tok[len(p):], 1.0)
        elp = torch.tensor([x[0] for x in r["meta_info"]["output_token_logprobs"]])
        assert torch.allclose(lp, elp, atol=atol)


@pytest.mark.parametrize("name", ["qwen3-tiny", "qwen3-tiny-moe"])
def test_prefix_cache_shares_prompt_pages_and_changes_nothing(name):
    """Eight samples of one prompt (the GRPO group), a second prompt, and a follow-up turn that re-sends a finished
    conversation: with the prefix cache the shared tokens are computed once, and tokens, log-probs and routed experts
    equal those of an engine without it."""
    cfg, m, plain = _engine(name, max_running=8, page_size=8, max_seq_len=160)
    _, _, cached = _engine(name, max_running=8, page_size=8, max_seq_len=160, prefix_cache=True)
    cached.model = m
    p0, p1 = _prompts(cfg, [37, 21], seed=3)
    prompts = [p0] * 4 + [p1] * 2
    sps = [SamplingParams(max_new_tokens=6 + i, sampling_seed=i) for i in range(len(prompts))]
    moe = cfg.is_moe
    a = plain.generate(prompts, sps, return_routed_experts=moe)
    b = cached.generate(prompts, sps, return_routed_experts=moe)
    for ra, rb in zip(a, b):
        assert ra["output_ids"] == rb["output_ids"]
        la = torch.tensor([x[0] for x in ra["meta_info"]["output_token_logprobs"]])
        lb = torch.tensor([x[0] for x in rb["meta_info"]["output_token_logprobs"]])
        assert torch.allclose(la, lb, atol=1e-5)
        if moe:
            assert torch.equal(ra["meta_info"]["routed_experts"], rb["meta_info"]["routed_experts"])
    _logprob_parity(m, prompts, b)
    # samples 2..4 of the first prompt found its four full pages (32 of 37 tokens), the second sample of the other its two
    assert [r["meta_info"]["cached_tokens"] for r in b] == [0, 32, 32, 32, 0, 16]
    assert cached.stats["prefill_tokens"] < plain.stats["prefill_tokens"]
    assert not cached.running and cached.pool.num_free + cached.prefix.num_pages == cached.num_pages - 1
    # a follow-up turn: the whole first conversation plus a few new tokens
    turn2 = p0 + b[0]["output_ids"] + _prompts(cfg, [5], seed=9)[0]
    ra = plain.generate([turn2], SamplingParams(max_new_tokens=5, sampling_seed=40), return_routed_experts=moe)[0]
    rb = cached.generate([turn2], SamplingParams(max_new_tokens=5, sampling_seed=40), return_routed_experts=moe)[0]
    assert ra["output_ids"] == rb["output_ids"] and rb["meta_info"]["cached_tokens"] >= 40
    if moe:
        assert torch.equal(ra["meta_info"]["routed_experts"], rb["meta_info"]["routed_experts"])
    # a weight update forgets everything
    assert cached.flush_cache() and cached.prefix.num_pages == 0 and cached.pool.num_free == cached.num_pages - 1
    rc = cached.generate([turn2], SamplingParams(max_new_tokens=5, sampling_seed=40))[0]
    assert rc["meta_info"]["cached_tokens"] == 0 and rc["output_ids"] == ra["output_ids"]


def test_prefix_cache_gives_pages_back_under_pressure():
    """A pool too small to keep everything cached: unreferenced cached pages are evicted, nothing leaks, results hold."""
    cfg, m, eng = _engine(max_running=2, page_size=8, max_seq_len=64, num_pages=14, prefix_cache=True)
    prompts = _prompts(cfg, [30, 28, 33, 31, 29, 27], seed=5)
    sps = [SamplingParams(max_new_tokens=10, sampling_seed=i) for i in range(len(prompts))]
    res = eng.generate(prompts, sps)
    assert [len(r["output_ids"]) for r in res] == [10] * 6
    _logprob_parity(m, prompts, res)
    assert eng.pool.num_free + eng.prefix.num_pages == eng.num_pages - 1


def test_sampling_parameters_that_are_not_built_are_refused_not_dropped():
    import pytest

    from miles_b200.engine.core import SamplingParams

    ok = SamplingParams.from_dict({"temperature": 0.7, "top_p": 0.9, "skip_special_tokens": True, "repetition_penalty": 1.0, "min_p": 0.0,
                                   "n": 1, "stop_token_ids": [3]})
    assert ok.temperature == 0.7 and ok.stop_token_ids == (3,)
    for bad in ({"repetition_penalty": 1.1}, {"min_p": 0.05}, {"presence_penalty": 0.5}, {"json_schema": "{}"}, {"n": 4}):
        with pytest.raises(ValueError):
            SamplingParams.from_dict(bad)
    from fastapi.testclient import TestClient

    from miles_b200.engine.server import build_app

    cfg, m, eng = _engine()
    with TestClient(build_app(eng)) as c:
        r = c.post("/generate", json={"input_ids": [1, 2, 3], "sampling_params": {"max_new_tokens": 2, "min_p": 0.1}})
        assert r.status_code == 400 and "min_p" in r.text
        assert c.post("/generate", json={"input_ids": [1, 2, 3], "sampling_params": {"max_new_tokens": 2}}).status_code == 200


def test_default_sampling_seeds_follow_the_salt_not_the_process():
    """Requests without a seed draw from (salt, request id): the same salt reproduces a run in any process, another salt
    (another --seed, another rank) samples differently."""
    cfg, m, a = _engine()
    _, _, b = _engine()
    _, _, c = _engine()
    a.seed_salt = b.seed_salt = 1234 * 1000003
    c.seed_salt = 1234 * 1000003 + 1
    prompts = _prompts(cfg, [12, 9], seed=4)
    sp = SamplingParams(max_new_tokens=12, temperature=1.0)
    ra, rb, rc = (e.generate(prompts, sp) for e in (a, b, c))
    assert [r["output_ids"] for r in ra] == [r["output_ids"] for r in rb]
    assert [r["output_ids"] for r in ra] != [r["output_ids"] for r in rc]
