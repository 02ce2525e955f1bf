"""sm_100a model path vs the PyTorch fp32 autograd oracle: log-probs, entropy and every gradient."""
import pytest
import torch

from miles_b200.models import ParamStore, build_model, get_config

pytestmark = pytest.mark.gpu


def _batch(cfg, lens, dev, seed=0):
    g = torch.Generator().manual_seed(seed)
    T = sum(lens)
    tokens = torch.randint(0, cfg.vocab_size, (T,), generator=g).to(dev)
    pos = torch.cat([torch.arange(l) for l in lens]).to(dev)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=dev)
    rows, tg = [], []
    off = 0
    for l in lens:
        p = l // 3
        rows.append(torch.arange(off + p - 1, off + l - 1))
        tg.append(tokens[off + p: off + l].cpu())
        off += l
    return tokens.int(), pos.int(), cu, torch.cat(rows).to(dev), torch.cat(tg).to(dev)


@pytest.mark.parametrize("name", ["qwen3-smoke", "qwen3-smoke-moe", "llama3-smoke", "mixtral-smoke", "glm4moe-smoke", "glm4-smoke", "qwen2moe-smoke"])
def test_forward_backward_matches_autograd(name):
    dev = torch.device("cuda")
    cfg = get_config(name)
    store = ParamStore(cfg, dev, torch.bfloat16, init_std=0.05, seed=7)
    # give the norm weights some structure so their gradients are exercised
    for n, p in store.named_parameters():
        if n.endswith("norm.weight") or ".ln" in n:
            p.add_(torch.randn_like(p) * 0.1)
    store.allocate_grads(torch.float32)
    model = build_model(cfg, store, "b200")
    ref_store = ParamStore(cfg, dev, torch.float32, init=False)
    ref_store.copy_from(store)
    ref = build_model(cfg, ref_store, "torch")
    ref.set_requires_grad(True)

    tokens, pos, cu, rows, tg = _batch(cfg, [200, 333, 75], dev)
    inv_temp = 1.0 / 0.9
    coef = torch.randn(rows.numel(), device=dev)

    def loss_fn(lp, ent):
        loss = (lp * coef).sum() / 50 + 0.01 * ent.sum()
        return loss, {}

    record = []
    lp0, ent0 = model.forward_logprobs(tokens, pos, cu, rows, tg, inv_temp, record=record)
    replay = torch.stack(record, 1) if record else None
    loss, _, lp, ent = model.forward_backward(tokens, pos, cu, rows, tg, inv_temp, loss_fn, replay=replay)
    model.check_status()
    assert torch.allclose(lp0, lp, atol=1e-5)

    rlp, rent = ref.forward_logprobs(tokens, pos, cu, rows, tg, inv_temp, replay=replay, with_grad=True)
    rloss, _ = loss_fn(rlp, rent)
    rloss.backward()
    assert (lp - rlp).abs().mean().item() < 0.02, (lp - rlp).abs().mean().item()
    assert (ent - rent).abs().mean().item() < 0.02
    bad = []
    for g in ("dense", "expert"):
        if store.flat[g].numel() == 0:
            continue
    for s in store.specs:
        got = store.grads[s.name].float()
        want = ref_store.flat[s.group].grad[s.offset:s.offset + s.numel].view(s.shape)
        denom = want.abs().max().item() + 1e-6
        rel = (got - want).abs().max().item() / denom            # worst element against the gradient's scale
        l2 = (got - want).norm().item() / (want.norm().item() + 1e-12)
        cos = torch.nn.functional.cosine_similarity(got.flatten(), want.flatten(), dim=0).item() if want.abs().sum() > 0 else 1.0
        # bf16 activations against an fp32 autograd reference: direction, overall size and the worst element
        if cos < 0.99 or l2 > 0.12 or rel > 0.25:
            bad.append((s.name, round(rel, 4), round(l2, 4), round(cos, 5)))
    assert not bad, bad


def test_replay_changes_nothing_when_ids_match():
    dev = torch.device("cuda")
    cfg = get_config("qwen3-smoke-moe")
    store = ParamStore(cfg, dev, torch.bfloat16, init_std=0.05)
    model = build_model(cfg, store, "b200")
    tokens, pos, cu, rows, tg = _batch(cfg, [128, 64], dev, seed=3)
    rec = []
    lp, _ = model.forward_logprobs(tokens, pos, cu, rows, tg, 1.0, record=rec)
    lp2, _ = model.forward_logprobs(tokens, pos, cu, rows, tg, 1.0, replay=torch.stack(rec, 1))
    assert torch.equal(lp, lp2)
