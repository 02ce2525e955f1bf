"""Helper launched by torchrun (2+ GPUs): the peer-memory weight push against plain slicing / the stand-alone quantisers.

    torchrun --nproc-per-node 2 tests/mp_weight_push_check.py check      # layouts and formats, bitwise
    torchrun --nproc-per-node 2 tests/mp_weight_push_check.py timing     # experts of a few 30B-A3B layers vs NCCL all-gather
"""
import copy
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist

from miles_b200.models import ParamStore, get_config
from miles_b200.ops.mx_gemm import quantize_operand
from miles_b200.parallel.state import init_parallel_state
from miles_b200.weight_sync.p2p_push import Layout, PushTarget, WeightPusher


def expect_equal(got: ParamStore, want: ParamStore, groups):
    for s in want.specs:
        if s.group in groups:
            assert torch.equal(got.params[s.name], want.params[s.name]), s.name


def check(ps, dev):
    world, rank = ps.world_size, ps.rank
    group = ps.world_group if hasattr(ps, "world_group") else None
    # A: expert-parallel trainer -> full expert replica on every GPU (bf16), dense shared by address
    cfg = get_config("qwen3-smoke-moe")
    src = ParamStore(cfg, dev, torch.bfloat16, ep_size=world, ep_rank=rank, seed=5)
    full = ParamStore(cfg, dev, torch.bfloat16, seed=5)
    for quant in ("none", "mxfp8", "nvfp4"):
        tgt = PushTarget.create(cfg, group, rank, world, dev, groups=("expert",), quant=quant, share_dense=src)
        pusher = WeightPusher(cfg, src, tgt, rank, [Layout(ep_size=world, ep_rank=r) for r in range(world)],
                              [Layout() for _ in range(world)], skip_groups=("dense",) if quant == "none" else ())
        for version in (1, 2):   # twice: flags and counters are reused
            if version == 2:
                for p in src.params.values():
                    p.mul_(0.5)
                for p in full.params.values():
                    p.mul_(0.5)
            pusher.push(version)
            torch.cuda.synchronize()
            pusher.check_status()
            dist.barrier()
            expect_equal(tgt.store, full, ("expert",))
            for name, op in tgt.mx.items():
                w = full.params[name]
                ref = quantize_operand(w.reshape(-1, w.shape[-1]), quant)
                assert torch.equal(op.q, ref.q), (quant, name, "values")
                assert torch.equal(op.atoms, ref.atoms), (quant, name, "scales")
                if quant == "nvfp4":
                    assert torch.allclose(torch.as_tensor(op.decode_scale).float().cpu(), torch.as_tensor(ref.decode_scale).float().cpu())
        if quant != "none":
            assert len(tgt.mx) >= 4, len(tgt.mx)
        src = ParamStore(cfg, dev, torch.bfloat16, ep_size=world, ep_rank=rank, seed=5)
        full = ParamStore(cfg, dev, torch.bfloat16, seed=5)
        dist.barrier()
    # B: tensor-parallel trainer -> unsharded engine on every GPU
    cfg = get_config("qwen3-smoke")
    src = ParamStore(cfg, dev, torch.bfloat16, tp_size=world, tp_rank=rank, seed=7)
    full = ParamStore(cfg, dev, torch.bfloat16, seed=7)
    tgt = PushTarget.create(cfg, group, rank, world, dev, groups=("dense",), quant="mxfp8")
    pusher = WeightPusher(cfg, src, tgt, rank, [Layout(tp_size=world, tp_rank=r) for r in range(world)], [Layout() for _ in range(world)])
    pusher.push()
    torch.cuda.synchronize()
    pusher.check_status()
    dist.barrier()
    expect_equal(tgt.store, full, ("dense",))
    for name, op in tgt.mx.items():
        ref = quantize_operand(full.params[name], "mxfp8")
        assert torch.equal(op.q, ref.q) and torch.equal(op.atoms, ref.atoms), name
    assert len(tgt.mx) == 4 * cfg.num_layers, len(tgt.mx)
    # C: replicated (data-parallel) trainer -> tensor-parallel engine, shard r on GPU r: every GPU serves itself
    src = ParamStore(cfg, dev, torch.bfloat16, seed=7)
    want = ParamStore(cfg, dev, torch.bfloat16, tp_size=world, tp_rank=rank, seed=7)
    tgt = PushTarget.create(cfg, group, rank, world, dev, groups=("dense",), tp_size=world, tp_rank=rank)
    pusher = WeightPusher(cfg, src, tgt, rank, [Layout() for _ in range(world)], [Layout(tp_size=world, tp_rank=r) for r in range(world)])
    assert pusher.src_mask == 1 << rank and pusher.flag_mask == 1 << rank
    pusher.push()
    torch.cuda.synchronize()
    pusher.check_status()
    expect_equal(tgt.store, want, ("dense",))
    dist.barrier()
    # D: a source that never arrives: the bounded wait gives up, records the status and the context stays usable
    pusher.C.weight_push_wait(tgt.flags_addr, 1 << ((rank + 1) % world), 10 ** 9, 30.0, pusher.status)
    torch.cuda.synchronize()
    try:
        pusher.check_status()
        raise AssertionError("the wait should have expired")
    except RuntimeError as e:
        assert "never arrived" in str(e)
    assert float(torch.ones(4, device=dev).sum()) == 4.0
    dist.barrier()


def timing(ps, dev, layers=4, iters=5):
    world, rank = ps.world_size, ps.rank
    cfg = copy.copy(get_config("qwen3-30B-A3B"))
    cfg.num_layers = layers
    src = ParamStore(cfg, dev, torch.bfloat16, ep_size=world, ep_rank=rank, seed=3)
    out = {"what": "weight_push", "world": world, "layers": layers}
    for quant in ("none", "mxfp8", "nvfp4"):
        tgt = PushTarget.create(cfg, None, rank, world, dev, groups=("expert",), quant=quant, share_dense=src, build_store=(quant == "none"))
        pusher = WeightPusher(cfg, src, tgt, rank, [Layout(ep_size=world, ep_rank=r) for r in range(world)], [Layout() for _ in range(world)],
                              skip_groups=("dense",))
        ms = []
        for it in range(iters + 2):
            dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            pusher.push()
            e1.record()
            torch.cuda.synchronize()
            pusher.check_status()
            t = torch.tensor([e0.elapsed_time(e1)], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            if it >= 2:
                ms.append(float(t))
        expert_bytes = src.flat["expert"].numel() * 2
        best = sorted(ms)[len(ms) // 2]
        out[f"push_{quant}_ms"] = best
        out[f"push_{quant}_src_GBps"] = expert_bytes / best / 1e6                      # shard bytes read per second
        out[f"push_{quant}_nvlink_out_GBps"] = expert_bytes * (world - 1) * {"none": 1.0, "mxfp8": 33 / 64, "nvfp4": 9 / 32}[quant] / best / 1e6
        if quant == "none":
            # the library path: all-gather of every expert tensor into the replica
            from miles_b200.weight_sync.reshard import gather_experts_into
            ms2 = []
            for it in range(iters + 2):
                dist.barrier()
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                gather_experts_into(src, tgt.store, None)
                e1.record()
                torch.cuda.synchronize()
                t = torch.tensor([e0.elapsed_time(e1)], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                if it >= 2:
                    ms2.append(float(t))
            out["nccl_all_gather_ms"] = sorted(ms2)[len(ms2) // 2]
        out["expert_shard_GB"] = expert_bytes / 1e9
        tgt.region.close()
        del tgt, pusher
        torch.cuda.empty_cache()
        dist.barrier()
    if rank == 0:
        print(json.dumps(out), flush=True)


def main():
    mode = sys.argv[1]
    world = int(os.environ["WORLD_SIZE"])
    ps = init_parallel_state(ep=world)
    dev = ps.device
    if mode == "check":
        check(ps, dev)
        if ps.rank == 0:
            print(f"WEIGHT_PUSH_CHECK_OK world={world}")
    else:
        timing(ps, dev, layers=int(sys.argv[2]) if len(sys.argv) > 2 else 4)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
