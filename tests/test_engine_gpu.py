"""Rollout engine on the GPU: trainer/rollout log-prob parity (eager and CUDA-graph decode), paged decode
attention vs a PyTorch reference, sampling kernel statistics."""
import math

import pytest
import torch

from miles_b200.engine import Engine, SamplingParams
from miles_b200.models import ParamStore, build_model, get_config
from miles_b200.ops import reference as R

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", ["qwen3-smoke", "qwen3-smoke-moe", "llama3-smoke", "mixtral-smoke", "glm4moe-smoke", "glm4-smoke", "qwen2moe-smoke"])
@pytest.mark.parametrize("graph", [False, True])
def test_engine_trainer_logprob_parity(name, graph):
    dev = torch.device("cuda")
    cfg = get_config(name)
    st = ParamStore(cfg, dev, torch.bfloat16, init_std=0.02)
    m = build_model(cfg, st, "b200")
    eng = Engine(m, max_running=8, page_size=64, max_seq_len=512, use_cuda_graph=graph)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (100, 37, 64, 5, 130)]
    sps = [SamplingParams(temperature=1.0, max_new_tokens=n, sampling_seed=i) for i, n in enumerate((40, 70, 12, 33, 90))]
    res = eng.generate(prompts, sps, return_routed_experts=True)
    for p, r, sp in zip(prompts, res, sps):
        assert len(r["output_ids"]) == sp.max_new_tokens
        ids = p + r["output_ids"]
        tok = torch.tensor(ids, dtype=torch.int32, device=dev)
        pos = torch.arange(len(ids), dtype=torch.int32, device=dev)
        cu = torch.tensor([0, len(ids)], dtype=torch.int32, device=dev)
        rows = torch.arange(len(p) - 1, len(ids) - 1, device=dev)
        replay = None
        if cfg.is_moe:
            re = r["meta_info"]["routed_experts"].to(dev)
            assert re.shape[0] == len(ids) - 1
            replay = torch.cat([re, re[-1:]], 0)
        lp, _ = m.forward_logprobs(tok, pos, cu, rows, tok[len(p):], 1.0, replay=replay)
        elp = torch.tensor([x[0] for x in r["meta_info"]["output_token_logprobs"]], device=dev)
        assert (lp - elp).abs().mean().item() < 0.01, (graph, (lp - elp).abs().mean().item())
    m.check_status()


def test_paged_decode_attention_matches_reference(ext):
    dev = torch.device("cuda")
    torch.manual_seed(0)
    B, Hq, Hk, D, ps = 5, 32, 4, 128, 64
    lens = [1, 63, 64, 200, 1000]
    max_pages = 20
    n_pages = 1 + sum((l + ps - 1) // ps for l in lens)
    kc = torch.randn(n_pages * ps, Hk, D, device=dev, dtype=torch.bfloat16)
    vc = torch.randn(n_pages * ps, Hk, D, device=dev, dtype=torch.bfloat16)
    bt = torch.zeros(B, max_pages, dtype=torch.int32, device=dev)
    nxt = 1
    for b, l in enumerate(lens):
        n = (l + ps - 1) // ps
        bt[b, :n] = torch.arange(nxt, nxt + n, dtype=torch.int32)
        nxt += n
    q = torch.randn(B, Hq, D, device=dev, dtype=torch.bfloat16)
    sl = torch.tensor(lens, dtype=torch.int32, device=dev)
    for splits in (1, 4, 16):
        out = torch.empty_like(q)
        scratch = torch.empty(B * Hq * splits * 130, dtype=torch.float32, device=dev)
        ext.paged_decode_attention(q, kc, vc, bt, sl, out, scratch, ps, splits, D ** -0.5)
        for b, l in enumerate(lens):
            slots = (bt[b, : (l + ps - 1) // ps].long()[:, None] * ps + torch.arange(ps, device=dev)[None]).reshape(-1)[:l]
            ref = R.attention_prefix(q[b:b + 1].float(), kc[slots].float(), vc[slots].float(), l - 1, D ** -0.5)
            assert (out[b].float() - ref[0]).abs().max().item() < 2e-2


def test_sampling_kernel_distribution(ext):
    dev = torch.device("cuda")
    torch.manual_seed(0)
    V, B = 1000, 4096
    base = torch.randn(V, device=dev) * 2
    logits = base[None].repeat(B, 1).contiguous()
    out = torch.empty(B, dtype=torch.int32, device=dev)
    lp = torch.empty(B, dtype=torch.float32, device=dev)
    seeds = torch.arange(B, dtype=torch.int64, device=dev) * 7919 + 13
    step = torch.zeros(B, dtype=torch.int32, device=dev)
    t = torch.full((B,), 0.8, device=dev)
    ext.sample_rows(logits, t, None, None, seeds, step, out, lp)
    ref_lp = torch.log_softmax(base / 0.8, -1)
    assert torch.allclose(lp, ref_lp[out.long()], atol=1e-4)
    # empirical frequencies of the most likely tokens match the softmax within sampling noise
    p = ref_lp.exp()
    top = p.topk(5).indices
    for i in top.tolist():
        f = (out == i).float().mean().item()
        assert abs(f - p[i].item()) < 5 * math.sqrt(p[i].item() / B) + 1e-3
    # top-k = 1 is argmax; top-p tiny is argmax too
    k1 = torch.ones(B, dtype=torch.int32, device=dev)
    ext.sample_rows(logits, t, k1, None, seeds, step, out, lp)
    assert (out == base.argmax()).all()
    pp = torch.full((B,), 1e-4, device=dev)
    ext.sample_rows(logits, t, None, pp, seeds, step, out, lp)
    assert (out == base.argmax()).all()
    # top-k = 10 never leaves the top-10 set
    k10 = torch.full((B,), 10, dtype=torch.int32, device=dev)
    ext.sample_rows(logits, t, k10, None, seeds, step, out, lp)
    allowed = set(base.topk(10).indices.tolist())
    assert set(out.tolist()) <= allowed
    # top-p = 0.5: sampled mass stays within the nucleus
    p5 = torch.full((B,), 0.5, device=dev)
    ext.sample_rows(logits, t, None, p5, seeds, step, out, lp)
    sp, si = p.sort(descending=True)
    nucleus = set(si[: int((sp.cumsum(0) < 0.5).sum().item()) + 1].tolist())
    assert set(out.tolist()) <= nucleus


@pytest.mark.parametrize("name", ["qwen3-smoke", "qwen3-smoke-moe"])
def test_prefix_cache_on_the_sm100_path(name):
    """The samples of one prompt share its pages (prefill of the later samples attends to cached keys / values through
    the tile table's key ranges), a follow-up turn finds the finished conversation; the log-probs the engine reports
    still match a recomputation with routing replay, and the routed experts of cached tokens come from the cache."""
    dev = torch.device("cuda")
    cfg = get_config(name)
    st = ParamStore(cfg, dev, torch.bfloat16, init_std=0.02)
    m = build_model(cfg, st, "b200")
    eng = Engine(m, max_running=8, page_size=64, max_seq_len=1024, use_cuda_graph=True, prefix_cache=True)
    g = torch.Generator().manual_seed(1)
    p0 = torch.randint(0, cfg.vocab_size, (300,), generator=g).tolist()
    p1 = torch.randint(0, cfg.vocab_size, (150,), generator=g).tolist()
    prompts = [p0] * 4 + [p1] * 2
    sps = [SamplingParams(temperature=1.0, max_new_tokens=30 + 7 * i, sampling_seed=i) for i in range(len(prompts))]
    res = eng.generate(prompts, sps, return_routed_experts=True)
    assert [r["meta_info"]["cached_tokens"] for r in res] == [0, 256, 256, 256, 0, 128]
    turn2 = p0 + res[0]["output_ids"] + torch.randint(0, cfg.vocab_size, (40,), generator=g).tolist()
    r2 = eng.generate([turn2], SamplingParams(temperature=1.0, max_new_tokens=20, sampling_seed=9), return_routed_experts=True)[0]
    assert r2["meta_info"]["cached_tokens"] >= 320
    m.check_status()
    for p, r in list(zip(prompts, res)) + [(turn2, r2)]:
        ids = p + r["output_ids"]
        tok = torch.tensor(ids, dtype=torch.int32, device=dev)
        pos = torch.arange(len(ids), dtype=torch.int32, device=dev)
        cu = torch.tensor([0, len(ids)], dtype=torch.int32, device=dev)
        rows = torch.arange(len(p) - 1, len(ids) - 1, device=dev)
        replay = None
        if cfg.is_moe:
            re = r["meta_info"]["routed_experts"].to(dev)
            assert re.shape[0] == len(ids) - 1
            replay = torch.cat([re, re[-1:]], 0)
        lp, _ = m.forward_logprobs(tok, pos, cu, rows, tok[len(p):], 1.0, replay=replay)
        elp = torch.tensor([x[0] for x in r["meta_info"]["output_token_logprobs"]], device=dev)
        d = (lp - elp).abs()
        assert d.mean().item() < 2e-2 and d.max().item() < 0.25, (d.mean().item(), d.max().item())
    assert not eng.running and eng.pool.num_free + eng.prefix.num_pages == eng.num_pages - 1


@pytest.mark.parametrize("name", ["qwen3-smoke", "qwen3-smoke-moe"])
def test_prefill_decode_hand_over_on_the_sm100_path(name):
    """Two engines on one model: the prompt's pages (and routed experts) move from the prefill engine's prefix cache to the
    decode engine's; the decode engine prefills only the tail, and the log-probs it reports match a recomputation."""
    from miles_b200.engine.pd import PDPair, pack_blob, unpack_blob

    dev = torch.device("cuda")
    cfg = get_config(name)
    st = ParamStore(cfg, dev, torch.bfloat16, init_std=0.02)
    m = build_model(cfg, st, "b200")
    prefill = Engine(m, max_running=4, page_size=64, max_seq_len=1024, use_cuda_graph=False, prefix_cache=True)
    decode = Engine(m, max_running=4, page_size=64, max_seq_len=1024, use_cuda_graph=True, prefix_cache=True)
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (300, 130)]
    sp = SamplingParams(temperature=1.0, max_new_tokens=24, sampling_seed=4)
    pair = PDPair(prefill, decode)
    res = pair.generate(prompts, sp, return_routed_experts=True)
    m.check_status()
    assert pair.transferred_tokens == 256 + 128
    assert [r["meta_info"]["cached_tokens"] for r in res] == [256, 128]
    assert decode.stats["prefill_tokens"] == (300 - 256) + (130 - 128)
    blob = prefill.export_prefix(prompts[0])
    back = unpack_blob(pack_blob(blob))                       # the byte form engines in other processes exchange
    assert torch.equal(back["kv"], blob["kv"]) and back["kv"].dtype == torch.bfloat16
    for p, r in zip(prompts, res):
        ids = p + r["output_ids"]
        tok = torch.tensor(ids, dtype=torch.int32, device=dev)
        pos = torch.arange(len(ids), dtype=torch.int32, device=dev)
        cu = torch.tensor([0, len(ids)], dtype=torch.int32, device=dev)
        rows = torch.arange(len(p) - 1, len(ids) - 1, device=dev)
        replay = None
        if cfg.is_moe:
            re = r["meta_info"]["routed_experts"].to(dev)
            assert re.shape[0] == len(ids) - 1
            replay = torch.cat([re, re[-1:]], 0)
        lp, _ = m.forward_logprobs(tok, pos, cu, rows, tok[len(p):], 1.0, replay=replay)
        elp = torch.tensor([x[0] for x in r["meta_info"]["output_token_logprobs"]], device=dev)
        d = (lp - elp).abs()
        assert d.mean().item() < 2e-2 and d.max().item() < 0.25, (d.mean().item(), d.max().item())
    for e in (prefill, decode):
        assert not e.running and e.pool.num_free + e.prefix.num_pages == e.num_pages - 1
