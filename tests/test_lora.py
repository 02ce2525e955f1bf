"""LoRA in merged form: adapter gradients equal autograd through the explicit low-rank path; only adapters move."""
import os

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


# ---------------------------------------------------------------------------------------------- tensor parallel
def _tp_lora_worker(rank: int, world: int, port: int, out_dir: str):
    """Each rank holds a tensor-parallel shard of the store and of the adapter; the weight gradients are the rank's slices of
    one full gradient. After two steps the gathered adapter must equal the adapter trained on the unsharded store."""
    import torch.distributed as dist

    from miles_b200.lora import LoRAManager
    from miles_b200.models import ParamStore, get_config
    from miles_b200.models.params import tp_slice

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        cfg = get_config("qwen3-tiny")
        dev = torch.device("cpu")
        full = ParamStore(cfg, dev, torch.float32, init_std=0.02, seed=3)
        full.allocate_grads(torch.float32)
        shard = ParamStore(cfg, dev, torch.float32, init_std=0.02, seed=3, tp_size=world, tp_rank=rank)
        shard.allocate_grads(torch.float32)
        for n, p in shard.params.items():      # same model: the shard is the slice of the full weights
            assert torch.equal(p, tp_slice(cfg, n, full.params[n], world, rank)), n
        ref = LoRAManager(full, 4, 8.0, "all-linear", lr=1e-2, seed=5)
        mine = LoRAManager(shard, 4, 8.0, "all-linear", lr=1e-2, seed=5, tp_group=dist.group.WORLD)
        assert sum(1 for t in mine.targets if t.tp == "col") and sum(1 for t in mine.targets if t.tp == "row")
        g = torch.Generator().manual_seed(11)
        for step in range(2):
            for n, gr in full.grads.items():
                gr.copy_(torch.randn(gr.shape, generator=g) * 0.1)
                shard.grads[n].copy_(tp_slice(cfg, n, gr, world, rank))
            ref.grads_from_weight_grads()
            mine.grads_from_weight_grads()
            n_ref, n_mine = ref.step(clip_grad=0.5), mine.step(clip_grad=0.5)
            assert abs(float(n_ref) - float(n_mine)) < 1e-5 * max(1.0, float(n_ref)), (step, float(n_ref), float(n_mine))
        want, got = ref.state_dict(), mine.state_dict()
        assert want.keys() == got.keys()
        for k in want:
            assert want[k].shape == got[k].shape, k
            # the all-reduce adds the partial gradients in another order than the unsharded product; Adam's normalised step
            # turns that rounding into a visible difference only where a gradient element is next to zero
            d = (want[k] - got[k]).abs()
            assert (d > 1e-5).float().mean().item() < 0.01 and d.max().item() < 2e-3, (k, d.max().item())
        for n, p in shard.params.items():      # merged weights: the slice of the unsharded merge
            assert (p - tp_slice(cfg, n, full.params[n], world, rank)).abs().max().item() < 1e-3, n
        # PEFT round trip through files: every rank gathers, rank 0 writes, a fresh sharded manager loads its slices
        d = os.path.join(out_dir, "adapter")
        mine.save(d, "base", write_adapter=rank == 0)
        dist.barrier()
        assert os.path.exists(os.path.join(d, f"training_state_tp{rank}.pt"))
        again = LoRAManager(shard, 4, 8.0, "all-linear", lr=1e-2, seed=99, tp_group=dist.group.WORLD, base=mine.base)
        again.load(d)
        for a, b in zip(again.A + again.B, mine.A + mine.B):
            assert torch.equal(a, b)
    finally:
        dist.destroy_process_group()


def test_adapter_under_tensor_parallelism_equals_the_unsharded_adapter(tmp_path):
    import socket

    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_tp_lora_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
