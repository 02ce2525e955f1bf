"""Helper launched by torchrun (2 GPUs): a two-stage pipeline (1F1B) vs the same model on one rank."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist

from miles_b200.models import ParamStore, build_model, get_config
from miles_b200.parallel.pipeline_parallel import PipeGroup, PipelineSchedule
from miles_b200.parallel.state import init_parallel_state


def make_mb(cfg, dev, seed, lens):
    g = torch.Generator().manual_seed(seed)
    T = sum(lens)
    tokens = torch.randint(0, cfg.vocab_size, (T,), generator=g).to(dev).int()
    pos = torch.cat([torch.arange(l) for l in lens]).to(dev).int()
    starts = [0]
    for l in lens:
        starts.append(starts[-1] + l)
    cu = torch.tensor(starts, dtype=torch.int32, device=dev)
    rows = torch.cat([torch.arange(a + 2, a + l - 1) for a, l in zip(starts, lens)]).to(dev)
    tg = tokens[(rows + 1).long()]
    coef = torch.randn(rows.numel(), generator=g).to(dev)
    return dict(tokens=tokens, pos=pos, cu=cu, rows=rows, tg=tg, coef=coef, max_seqlen=max(lens))


def main():
    world = int(os.environ["WORLD_SIZE"])
    ps = init_parallel_state(pp=world)
    dev = ps.device
    for preset in ("qwen3-smoke", "qwen3-smoke-moe"):
        cfg = get_config(preset)
        store = ParamStore(cfg, dev, torch.bfloat16, init_std=0.05, seed=5, pp_size=world, pp_rank=ps.pp.rank)
        store.allocate_grads(torch.float32)
        model = build_model(cfg, store, "b200")
        ref_store = ParamStore(cfg, dev, torch.bfloat16, init_std=0.05, seed=5)
        ref_store.allocate_grads(torch.float32)
        ref = build_model(cfg, ref_store, "b200")
        for name, t in store.params.items():
            assert torch.equal(t, ref_store.params[name]), name
        mbs = [make_mb(cfg, dev, 20 + i, lens) for i, lens in enumerate([[90, 41], [150], [33, 60, 70], [128]])]
        loss_of = lambda mb: (lambda lp, ent: ((lp * mb["coef"]).sum() / 40 + 0.01 * ent.sum(), {}))
        # reference: plain loop over the micro-batches
        lp_ref = []
        for mb in mbs:
            _, _, lp, _ = ref.forward_backward(mb["tokens"], mb["pos"], mb["cu"], mb["rows"], mb["tg"], 1.0, loss_of(mb),
                                               max_seqlen=mb["max_seqlen"])
            lp_ref.append(lp)
        # pipeline
        sch = PipelineSchedule(PipeGroup(ps.pp.group, ps.pp.rank, world, ps.pp.ranks), dev)
        meta = lambda i: ((mbs[i]["tokens"].shape[0], cfg.hidden_size), torch.bfloat16)
        saved, lps = {}, {}
        last = store.is_last_stage

        def fwd(i, x_in):
            mb = mbs[i]
            if last:
                saved[i] = x_in
                return None
            inputs = []
            y = model.forward_hidden(mb["tokens"], mb["pos"], mb["cu"], max_seqlen=mb["max_seqlen"], save_inputs=inputs, x_in=x_in)
            inputs.pop()
            saved[i] = inputs
            return y

        def bwd(i, dy):
            mb = mbs[i]
            if last:
                _, _, lp, _ = model.forward_backward(mb["tokens"], mb["pos"], mb["cu"], mb["rows"], mb["tg"], 1.0, loss_of(mb),
                                                     max_seqlen=mb["max_seqlen"], x_in=saved.pop(i))
                lps[i] = lp
                return model.last_dx_in
            return model.layers_backward(saved.pop(i), dy, mb["tokens"], mb["pos"], mb["cu"], mb["max_seqlen"], None)

        sch.run_1f1b(len(mbs), meta, fwd, bwd)
        model.check_status()
        torch.cuda.synchronize()
        assert not saved
        if last:
            for i, lp in lps.items():
                assert torch.allclose(lp, lp_ref[i], atol=1e-3), (preset, i, (lp - lp_ref[i]).abs().max().item())
        for name, gr in store.grads.items():
            want = ref_store.grads[name]
            if want.abs().max().item() == 0:
                continue
            cos = torch.nn.functional.cosine_similarity(gr.flatten().float(), want.flatten().float(), dim=0).item()
            assert cos > 0.999, (preset, name, cos)
        # forward-only pipeline gives the reference log-probs on the last stage
        outs = {}

        def fwd_only(i, x_in):
            mb = mbs[i]
            if last:
                outs[i] = model.forward_logprobs(mb["tokens"], mb["pos"], mb["cu"], mb["rows"], mb["tg"], 1.0,
                                                 max_seqlen=mb["max_seqlen"], x_in=x_in)[0]
                return None
            return model.forward_hidden(mb["tokens"], mb["pos"], mb["cu"], max_seqlen=mb["max_seqlen"], x_in=x_in)

        sch.run_forward_only(len(mbs), meta, fwd_only)
        if last:
            for i, lp in outs.items():
                assert torch.allclose(lp, lp_ref[i], atol=1e-3), (preset, i)
        dist.barrier()
    if ps.rank == 0:
        print(f"PP_CHECK_OK world={world}")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
