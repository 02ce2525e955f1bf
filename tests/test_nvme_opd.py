"""File-backed Adam equals in-memory AdamW; on-policy-distillation advantage correction."""
import math

import torch

from miles_b200.models import ParamStore, get_config
from miles_b200.rl.opd import apply_opd, teacher_logprob_from_topk
from miles_b200.trainer.nvme_optimizer import NvmeStreamedAdam


def test_nvme_adam_matches_torch_adamw(tmp_path):
    cfg = get_config("qwen3-tiny")
    store = ParamStore(cfg, "cpu", torch.float32, seed=2)
    store.allocate_grads(torch.float32)
    ref = {g: t.clone().requires_grad_(True) for g, t in store.flat.items() if t.numel()}
    topt = torch.optim.AdamW(list(ref.values()), lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    opt = NvmeStreamedAdam(store, str(tmp_path), lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1, bucket_elems=50_000, moment_dtype="fp32")
    assert len(opt.buckets) > 3
    gen = torch.Generator().manual_seed(0)
    for _ in range(3):
        for g, t in ref.items():
            gr = torch.randn(t.shape, generator=gen) * 0.01
            store.grad[g].copy_(gr)
            t.grad = gr.clone()
        opt.step()
        topt.step()
    for g, t in ref.items():
        assert torch.allclose(store.flat[g], t.detach(), atol=2e-6, rtol=1e-5), g
    assert opt.bytes_read > 0 and opt.bytes_written > 0
    # a fresh optimizer over the same directory resumes from the files
    again = NvmeStreamedAdam(store, str(tmp_path), lr=1e-2, bucket_elems=50_000)
    m = again._load_bucket(0)[1]
    assert m.abs().sum() > 0


def test_opd_lowers_advantage_where_student_is_overconfident():
    adv = torch.zeros(4)
    s = torch.tensor([-0.1, -2.0, -1.0, -0.5])
    t = torch.tensor([-1.1, -2.0, -0.5, -0.5])
    out, kl = apply_opd(adv, s, t, opd_kl_coef=0.5, loss_mask=torch.tensor([1, 1, 1, 0]))
    assert torch.allclose(out, torch.tensor([-0.5, 0.0, 0.25, 0.0]))
    assert abs(float(kl) - (1.0 + 0.0 - 0.5) / 3) < 1e-6
    lp = teacher_logprob_from_topk(7, [1, 2], [math.log(0.5), math.log(0.3)], vocab_size=12)
    assert abs(lp - math.log(0.2 / 10)) < 1e-9
    assert teacher_logprob_from_topk(2, [1, 2], [math.log(0.5), math.log(0.3)], 12) == math.log(0.3)


def _teacher_post(teacher_client):
    """Stands in for the HTTP hop: the payload goes straight to an in-process teacher engine's /generate handler."""
    async def post(url, payload):
        assert url.startswith("http://teacher-"), url
        post.calls.append(url)
        return await teacher_client.generate(payload)
    post.calls = []
    return post


def test_engine_scores_a_sequence_like_the_trainer():
    from miles_b200.engine import Engine
    from miles_b200.models import build_model

    cfg = get_config("qwen3-tiny")
    m = build_model(cfg, ParamStore(cfg, "cpu", torch.float32, seed=3))
    eng = Engine(m, max_running=2, page_size=8, max_seq_len=64)
    ids = torch.randint(0, cfg.vocab_size, (23,), generator=torch.Generator().manual_seed(1)).tolist()
    out = eng.score(ids, top_k=4)
    tok, pos, cu = torch.tensor(ids), torch.arange(23), torch.tensor([0, 23])
    lp, _ = m.forward_logprobs(tok, pos, cu, torch.arange(0, 22), tok[1:], 1.0)
    assert out["logprobs"][0] is None and torch.allclose(torch.tensor(out["logprobs"][1:]), lp, atol=1e-5)
    assert out["top"][0] is None and len(out["top"][5]["ids"]) == 4
    assert out["top"][5]["logprobs"][0] >= out["logprobs"][5] - 1e-6          # the best token is at least as likely
    assert torch.allclose(torch.tensor(eng.score(ids)["logprobs"][1:]), lp, atol=1e-5)


def test_remote_teacher_distillation_through_the_loop():
    """--use-opd --opd-type sglang: every generated sample is scored by the teacher its metadata names (or the default),
    the teacher's log-probs reach the trainer, and the advantages carry the per-token penalty."""
    import asyncio

    from miles_b200.engine import Engine
    from miles_b200.engine.client import EngineClient
    from miles_b200.loop import RLLoop
    from miles_b200.models import build_model
    from miles_b200.rollout.on_policy_distillation import parse_teacher_urls, teacher_url_for_sample
    from miles_b200.utils.arguments import parse_args
    from miles_b200.utils.types import Sample

    import pytest
    with pytest.raises(ValueError):
        parse_teacher_urls(["no-equals-sign"])
    with pytest.raises(ValueError):
        parse_teacher_urls(["a=http://x", "a=http://y"])
    base = ["--model-preset", "qwen3-tiny", "--rollout-batch-size", "4", "--n-samples-per-prompt", "2", "--rollout-max-response-len", "8",
            "--rollout-max-prompt-len", "16", "--lr", "1e-5", "--micro-batch-size", "8", "--colocate", "--num-rollout", "1",
            "--actor-num-gpus-per-node", "1", "--use-opd", "--opd-type", "sglang", "--opd-kl-coef", "0.5",
            "--opd-teacher-urls", "default=http://teacher-a/generate", "math=http://teacher-b/generate?x=1"]
    args = parse_args(base)
    s = Sample(index=0, prompt="p", metadata={"opd_teacher": "math"})
    assert teacher_url_for_sample(args, s) == "http://teacher-b/generate?x=1"
    s.metadata = {"opd_teacher": "unknown"}
    assert teacher_url_for_sample(args, s) == "http://teacher-a/generate"
    loop = RLLoop(args)
    cfg = loop.actor.cfg
    teacher = Engine(build_model(cfg, ParamStore(cfg, "cpu", torch.float32, seed=99)), max_running=2, page_size=8, max_seq_len=64)
    post = _teacher_post(EngineClient([teacher], None))
    loop.rollout_fn.state.teacher_post = post
    samples, _ = loop.generate(0)
    assert len(samples) == 8 and len(post.calls) == 8 and set(post.calls) == {"http://teacher-a/generate"}
    for sm in samples:
        assert len(sm.teacher_log_probs) == sm.response_length and sm.reward == 0.0
        ids = list(sm.tokens)
        want = teacher.score(ids)["logprobs"][-sm.response_length:]
        assert torch.allclose(torch.tensor(sm.teacher_log_probs), torch.tensor(want), atol=1e-5)
    if args.offload_train:
        loop.actor.wake_up()  # what RLLoop.step does before training
    m = loop.train(0, samples)
    assert m["train/grad_norm"] > 0  # zero task reward: the gradient comes from the distillation penalty alone
    # top-k scoring: tokens outside the teacher's top-k get the floor log-prob
    args2 = parse_args(base + ["--opd-log-prob-top-k", "3", "--opd-top-k-strategy", "only-teacher"])
    from miles_b200.rollout.on_policy_distillation import fetch_teacher_log_probs
    sm = samples[0]
    sm.teacher_log_probs = None
    asyncio.run(fetch_teacher_log_probs(args2, sm, post=post, vocab_size=cfg.vocab_size))
    exact = teacher.score(list(sm.tokens))["logprobs"][-sm.response_length:]
    assert len(sm.teacher_log_probs) == sm.response_length
    assert all(a <= 1e-6 and (abs(a - b) < 1e-5 or a < -3.0) for a, b in zip(sm.teacher_log_probs, exact))
