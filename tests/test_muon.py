"""Muon optimizer: Newton-Schulz orthogonalisation, parameter partition, training progress and state round trip (CPU)."""
import torch

from miles_b200.models import ParamStore, get_config
from miles_b200.trainer.muon import Muon, MuonConfig, is_muon_param, newton_schulz
from miles_b200.trainer.optimizer import OptimConfig


def test_newton_schulz_pushes_singular_values_towards_one():
    g = torch.Generator().manual_seed(0)
    for shape in ((64, 32), (32, 96), (3, 48, 48)):
        G = torch.randn(*shape, generator=g)
        O = newton_schulz(G, steps=8)
        sv = torch.linalg.svdvals(O.float())
        assert sv.max() < 1.3 and sv.min() > 0.5, (shape, sv.min().item(), sv.max().item())
        # the iteration keeps the singular vectors: O is close to U V^T of G
        U, _, Vh = torch.linalg.svd(G, full_matrices=False)
        assert torch.nn.functional.cosine_similarity((U @ Vh).flatten(), O.float().flatten(), dim=0) > 0.95


def test_parameter_partition():
    cfg = get_config("qwen3-tiny")
    store = ParamStore(cfg, "cpu", torch.float32, seed=1)
    muon = [n for n, p in store.params.items() if is_muon_param(n, tuple(p.shape))]
    assert all(n.startswith("layers.") for n in muon)
    assert "embed.weight" not in muon and not any("ln" in n or "norm" in n for n in muon)
    assert any(n.endswith("attn.qkv.weight") for n in muon) and any(n.endswith("mlp.down.weight") for n in muon)


def test_muon_step_reduces_a_quadratic_and_round_trips_state():
    cfg = get_config("qwen3-tiny")
    store = ParamStore(cfg, "cpu", torch.float32, seed=1)
    store.allocate_grads(torch.float32)
    target = {n: p.clone() + 0.05 * torch.randn_like(p) for n, p in store.params.items()}
    oc = OptimConfig(lr=2e-2, weight_decay=0.0, clip_grad=0.0, master_weights=False)
    opt = Muon(store, oc, MuonConfig(split_qkv=True))

    def loss_and_grads():
        tot = 0.0
        for n, p in store.params.items():
            d = p - target[n]
            store.grads[n].copy_(d)
            tot += float((d * d).sum())
        return tot

    l0 = loss_and_grads()
    for _ in range(20):
        gn = opt.step(1.0)
        l1 = loss_and_grads()
    assert torch.isfinite(gn) and l1 < 0.5 * l0, (l0, l1)
    # the Muon update of a matrix has (nearly) equal singular values: check one step in isolation
    name = next(n for n in opt.muon_names if n.endswith("mlp.down.weight"))
    before = store.params[name].clone()
    opt.momentum[name].zero_()
    opt.step(1.0)
    sv = torch.linalg.svdvals((store.params[name] - before).float())
    assert sv.max() / sv.min().clamp_min(1e-12) < 3.0
    sd = opt.state_dict()
    opt2 = Muon(store, oc)
    opt2.load_state_dict(sd)
    assert opt2.step_count == opt.step_count
    assert all(torch.equal(opt2.momentum[n], opt.momentum[n]) for n in opt.muon_names)


def test_non_finite_gradient_skips_the_step():
    cfg = get_config("qwen3-tiny")
    store = ParamStore(cfg, "cpu", torch.float32, seed=1)
    store.allocate_grads(torch.float32)
    opt = Muon(store, OptimConfig(lr=1e-2, master_weights=False))
    before = {n: p.clone() for n, p in store.params.items()}
    store.grads["embed.weight"].fill_(float("nan"))
    opt.step(1.0)
    assert all(torch.equal(before[n], p) for n, p in store.params.items())
