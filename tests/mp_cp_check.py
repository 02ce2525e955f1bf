"""Helper launched by torchrun (2 GPUs): context-parallel attention forward (zigzag shards, gathered K/V) vs one rank."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist

from miles_b200.ops import _ext
from miles_b200.ops.attention import attention_reference
from miles_b200.parallel.context_parallel import build_cp_tiles, gather_kv, gather_per_token, zigzag_slice
from miles_b200.parallel.state import init_parallel_state


def main():
    world = int(os.environ["WORLD_SIZE"])
    ps = init_parallel_state(cp=world)
    dev, C = ps.device, _ext.load(required=True)
    lens = [700, 129, 1500]
    T, Hq, Hk = sum(lens), 8, 2
    g = torch.Generator().manual_seed(4)
    qkv = torch.randn(T, Hq + 2 * Hk, 128, generator=g).to(dev).to(torch.bfloat16)
    q, k, v = qkv[:, :Hq].contiguous(), qkv[:, Hq:Hq + Hk].contiguous(), qkv[:, Hq + Hk:].contiguous()
    ref, _ = attention_reference(q, k, v, lens, 128 ** -0.5)
    ql, kl, vl = (zigzag_slice(t, lens, world, ps.cp.rank).contiguous() for t in (q, k, v))
    kf, vf = gather_kv(kl, vl, lens, world, ps.cp.group)
    assert torch.equal(kf, k) and torch.equal(vf, v)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    tiles = build_cp_tiles(lens, world, ps.cp.rank).to(dev)
    out_l, _ = C.flash_attn_fwd(ql, kf, vf, tiles, 128 ** -0.5, status)
    assert status.item() == 0
    out = gather_per_token(out_l.float(), lens, world, ps.cp.rank, ps.cp.group)
    rel = (out - ref).abs().max().item() / ref.abs().max().item()
    assert rel < 2e-2, rel
    if ps.rank == 0:
        print(f"CP_CHECK_OK world={world} rel={rel:.4f}")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
