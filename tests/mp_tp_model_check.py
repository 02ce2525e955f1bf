"""Helper launched by torchrun (2 GPUs): a tensor-parallel dense model vs the same model on one rank."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist

from miles_b200.models import ParamStore, build_model, get_config
from miles_b200.models.params import is_tp_sharded, tp_slice
from miles_b200.parallel.state import init_parallel_state
from miles_b200.parallel.tensor_parallel import TensorParallel


def main():
    fused = sys.argv[1] == "fused"
    world = int(os.environ["WORLD_SIZE"])
    ps = init_parallel_state(tp=world)
    dev = ps.device
    cfg = get_config("qwen3-smoke")
    store = ParamStore(cfg, dev, torch.bfloat16, init_std=0.05, seed=5, tp_size=world, tp_rank=ps.tp.rank)
    store.allocate_grads(torch.float32)
    tp = TensorParallel(ps.tp.group, ps.tp.rank, world, dev, cfg.hidden_size, 2048, fused=fused)
    model = build_model(cfg, store, "b200", tp=tp)
    ref_store = ParamStore(cfg, dev, torch.bfloat16, init_std=0.05, seed=5)
    ref_store.allocate_grads(torch.float32)
    ref = build_model(cfg, ref_store, "b200")
    for name, t in ref_store.params.items():
        assert torch.equal(tp_slice(cfg, name, t, world, ps.tp.rank), store.params[name]), name
    g = torch.Generator().manual_seed(11)
    lens = [90, 41, 150]
    T = sum(lens)
    tokens = torch.randint(0, cfg.vocab_size, (T,), generator=g).to(dev).int()
    pos = torch.cat([torch.arange(l) for l in lens]).to(dev).int()
    cu = torch.tensor([0, 90, 131, 281], dtype=torch.int32, device=dev)
    rows = torch.cat([torch.arange(a + 3, a + l - 1) for a, l in zip([0, 90, 131], lens)]).to(dev)
    tg = tokens[(rows + 1).long()]
    coef = torch.randn(rows.numel(), generator=g).to(dev)
    loss_fn = lambda lp, ent: ((lp * coef).sum() / 40 + 0.01 * ent.sum(), {})
    for it in range(2):
        store.zero_grads()
        ref_store.zero_grads()
        _, _, lp, _ = model.forward_backward(tokens, pos, cu, rows, tg, 1.0, loss_fn)
        _, _, lp_ref, _ = ref.forward_backward(tokens, pos, cu, rows, tg, 1.0, loss_fn)
        model.check_status()
        tp.check_status()
        d = (lp - lp_ref).abs()
        assert d.max().item() < 1e-1 and d.mean().item() < 2e-2, (d.max().item(), d.mean().item())  # partial sums are rounded to bf16 before they are added
        both = [torch.empty_like(lp) for _ in range(world)]
        dist.all_gather(both, lp)
        assert all(torch.equal(both[0], t) for t in both), "tensor-parallel ranks diverged"
        for name, gr in store.grads.items():
            want = ref_store.grads[name]
            if is_tp_sharded(name):
                want = tp_slice(cfg, name, want, world, ps.tp.rank)
            elif name.endswith(("q_norm.weight", "k_norm.weight")):
                gr = gr.clone()
                dist.all_reduce(gr)
            if want.abs().max().item() == 0:
                continue
            cos = torch.nn.functional.cosine_similarity(gr.flatten().float(), want.flatten().float(), dim=0).item()
            assert cos > 0.99, (name, cos)
    if ps.rank == 0:
        print(f"TP_MODEL_CHECK_OK fused={fused} world={world}")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
