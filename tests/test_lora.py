"""LoRA in merged form: adapter gradients equal autograd through the explicit low-rank path; only adapters move."""
import torch

from miles_b200.lora import LoRAManager
from miles_b200.models import ParamStore, build_model, get_config


def test_lora_gradients_match_explicit_low_rank(tmp_path):
    torch.manual_seed(0)
    cfg = get_config("qwen3-tiny")
    store = ParamStore(cfg, "cpu", torch.float32, seed=3)
    store.allocate_grads(torch.float32)
    model = build_model(cfg, store, "torch")
    lora = LoRAManager(store, rank=4, alpha=8, target_modules=["q_proj", "v_proj", "down_proj"], lr=1e-2)
    for b in lora.B:
        b.copy_(torch.randn_like(b) * 0.05)
    lora.merge()
    base = {n: t.clone() for n, t in lora.base.items()}
    T = 24
    tok = torch.randint(0, cfg.vocab_size, (T,))
    pos, cu = torch.arange(T), torch.tensor([0, T])
    rows, tg = torch.arange(3, T - 1), tok[4:]
    model.set_requires_grad(True)
    lp, _ = model.forward_logprobs(tok, pos, cu, rows, tg, 1.0, with_grad=True)
    (-lp.mean()).backward()
    model.accumulate_autograd_grads()
    model.set_requires_grad(False)
    lora.grads_from_weight_grads()
    # oracle: autograd through W = base + s * B @ A for one target
    t0 = lora.targets[0]
    A = lora.A[0].clone().requires_grad_(True)
    B = lora.B[0].clone().requires_grad_(True)
    dW = lora._slice(store.grads[t0.native], t0)
    ((lora.scale * (B @ A)) * dW).sum().backward()
    assert torch.allclose(lora.A[0].grad, A.grad, atol=1e-6) and torch.allclose(lora.B[0].grad, B.grad, atol=1e-6)
    before_A = lora.A[0].clone()
    lora.step(clip_grad=1.0)
    assert not torch.equal(before_A, lora.A[0])
    for n, b in base.items():
        assert torch.equal(lora.base[n], b)  # frozen base
    untouched = "layers.0.attn.o.weight"
    assert torch.equal(store.params[untouched], ParamStore(cfg, "cpu", torch.float32, seed=3).params[untouched])
    # PEFT round trip
    lora.save(str(tmp_path / "adapter"))
    lora2 = LoRAManager(ParamStore(cfg, "cpu", torch.float32, seed=3), rank=4, alpha=8, target_modules=["q_proj", "v_proj", "down_proj"])
    lora2.load(str(tmp_path / "adapter"))
    assert torch.equal(lora2.A[1], lora.A[1]) and torch.allclose(lora2.store.params[t0.native], store.params[t0.native])
    assert "base_model.model.model.layers.0.self_attn.q_proj.lora_A.weight" in lora.state_dict()
