"""Prefill / decode disaggregation: the prompt's keys / values travel from the prefill engine's prefix cache into the
decode engine's; a disaggregated run returns what the decode engine alone returns, and prefills only the tail there."""
import asyncio

import pytest
import torch

from miles_b200.engine import Engine, SamplingParams
from miles_b200.engine.pd import PDClient, PDPair, pack_blob, unpack_blob
from miles_b200.models import ParamStore, build_model, get_config


def _engine(name, **kw):
    cfg = get_config(name)
    st = ParamStore(cfg, "cpu", torch.float32, seed=11)
    m = build_model(cfg, st)
    kw.setdefault("max_running", 4)
    kw.setdefault("page_size", 8)
    kw.setdefault("max_seq_len", 160)
    return cfg, m, Engine(m, prefix_cache=True, **kw)


def _prompts(cfg, lens, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in lens]


@pytest.mark.parametrize("name", ["qwen3-tiny", "qwen3-tiny-moe"])
def test_handed_over_prefix_changes_nothing_but_the_prefill_work(name):
    cfg, m, alone = _engine(name)
    _, _, prefill = _engine(name)
    _, _, decode = _engine(name)
    prompts = _prompts(cfg, [37, 50, 9], seed=4)
    sps = SamplingParams(max_new_tokens=7, sampling_seed=5)
    moe = cfg.is_moe
    want = alone.generate(prompts, sps, return_routed_experts=moe)
    pair = PDPair(prefill, decode)
    got = pair.generate(prompts, sps, return_routed_experts=moe)
    for a, b in zip(want, got):
        assert a["output_ids"] == b["output_ids"]
        la = torch.tensor([x[0] for x in a["meta_info"]["output_token_logprobs"]])
        lb = torch.tensor([x[0] for x in b["meta_info"]["output_token_logprobs"]])
        assert torch.allclose(la, lb, atol=1e-5)
    # 4 + 6 + 1 full pages of 8 tokens crossed over; the decode engine prefilled only the tails
    assert pair.transferred_tokens == 32 + 48 + 8
    assert [r["meta_info"]["cached_tokens"] for r in got] == [32, 48, 8]
    assert decode.stats["prefill_tokens"] == (37 - 32) + (50 - 48) + (9 - 8)
    if moe:  # routing replay needs the routed experts of the prompt tokens too: they travel with the pages
        for a, b in zip(want, got):
            assert torch.equal(a["meta_info"]["routed_experts"], b["meta_info"]["routed_experts"])
    # no page leaked on either side
    for e in (prefill, decode):
        assert not e.running and e.pool.num_free + e.prefix.num_pages == e.num_pages - 1


def test_blob_round_trip_and_refusals():
    cfg, m, a = _engine("qwen3-tiny")
    _, _, b = _engine("qwen3-tiny")
    p = _prompts(cfg, [40], seed=1)[0]
    assert a.export_prefix(p) is None                       # nothing cached yet
    a.generate([p], SamplingParams(max_new_tokens=1, temperature=0.0))
    blob = a.export_prefix(p)
    assert len(blob["tokens"]) == 40 and blob["kv"].shape[:3] == (cfg.num_layers, 2, 40)
    back = unpack_blob(pack_blob(blob))
    assert back["tokens"] == blob["tokens"] and torch.equal(back["kv"], blob["kv"]) and back["page_size"] == 8
    assert unpack_blob(pack_blob(None)) is None
    with pytest.raises(ValueError):
        unpack_blob(b"something else")
    b.update_weight_version(3)
    assert b.import_prefix(back) == 0, "keys / values of another weight version are refused"
    b.update_weight_version(0)
    assert b.import_prefix(back) == 40
    assert b.import_prefix(back) == 40 and b.prefix.num_pages == 5, "importing twice keeps one copy"
    wrong = dict(back, page_size=16)
    assert b.import_prefix(wrong) == 0
    # a pool without room imports nothing and loses nothing
    _, _, small = _engine("qwen3-tiny", num_pages=4)
    assert small.import_prefix(back) == 0 and small.pool.num_free == 3


def test_http_endpoints_carry_the_hand_over():
    from fastapi.testclient import TestClient

    from miles_b200.engine.server import build_app

    cfg, m, alone = _engine("qwen3-tiny")
    _, _, prefill = _engine("qwen3-tiny")
    _, _, decode = _engine("qwen3-tiny")
    apps = {"http://p": TestClient(build_app(prefill)), "http://d": TestClient(build_app(decode))}

    async def transport(method, url, body):
        base, path = url[:8], url[8:]
        app = apps[base]
        if isinstance(body, (bytes, bytearray)):
            r = app.post(path, content=bytes(body), headers={"content-type": "application/octet-stream"})
        else:
            r = app.post(path, json=body)
        assert r.status_code == 200, r.text
        return r.content if path == "/export_prefix" else r.json()

    client = PDClient(["http://p"], ["http://d"], transport=transport)
    prompt = _prompts(cfg, [45], seed=8)[0]
    payload = {"input_ids": prompt, "sampling_params": {"max_new_tokens": 6, "sampling_seed": 9}}
    with apps["http://p"], apps["http://d"]:
        out = asyncio.run(client.generate(payload))
    want = alone.generate([prompt], SamplingParams(max_new_tokens=6, sampling_seed=9))[0]
    assert out["output_ids"] == want["output_ids"]
    assert client.transferred_tokens == 40 and out["meta_info"]["cached_tokens"] == 40


def test_remote_client_hands_over_before_every_request():
    """The rollout's HTTP client with ``prefill_urls``: /generate goes to decode engines only, control calls to all."""
    from fastapi.testclient import TestClient

    from miles_b200.engine.remote import RemoteEngineClient
    from miles_b200.engine.server import build_app

    cfg, m, alone = _engine("qwen3-tiny")
    engines = {"http://p": _engine("qwen3-tiny")[2], "http://d": _engine("qwen3-tiny")[2]}
    apps = {u: TestClient(build_app(e)) for u, e in engines.items()}
    calls = []

    async def transport(method, url, body):
        base, path = url[:8], url[8:]
        calls.append((base, path))
        if isinstance(body, (bytes, bytearray)):
            r = apps[base].post(path, content=bytes(body), headers={"content-type": "application/octet-stream"})
        elif method == "GET":
            r = apps[base].get(path)
        else:
            r = apps[base].post(path, json=body)
        out = r.content if path == "/export_prefix" else (r.json() if r.content else None)
        return (r.status_code, out) if not isinstance(body, (bytes, bytearray)) and path not in ("/export_prefix",) else out

    client = RemoteEngineClient(["http://p", "http://d"], transport=transport, prefill_urls=["http://p"])
    assert client.urls == ["http://d"]
    prompts = _prompts(cfg, [33, 20], seed=2)

    async def run():
        outs = []
        for i, p in enumerate(prompts):
            outs.append(await client.generate({"input_ids": p, "sampling_params": {"max_new_tokens": 5, "sampling_seed": i}}))
        await client.flush_cache()
        return outs

    with apps["http://p"], apps["http://d"]:
        outs = asyncio.run(run())
    want = [alone.generate([p], SamplingParams(max_new_tokens=5, sampling_seed=i))[0] for i, p in enumerate(prompts)]
    assert [o["output_ids"] for o in outs] == [w["output_ids"] for w in want]
    assert client.transferred_tokens == 32 + 16 and [o["meta_info"]["cached_tokens"] for o in outs] == [32, 16]
    assert ("http://p", "/generate") in calls and ("http://d", "/import_prefix") in calls
    assert {b for b, p in calls if p == "/flush_cache"} == {"http://p", "http://d"}
    assert engines["http://p"].prefix.num_pages == 0 and engines["http://d"].prefix.num_pages == 0  # flushed on both
