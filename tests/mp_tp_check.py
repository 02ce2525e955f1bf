"""Helper launched by torchrun (2+ GPUs): fused GEMM + partial-sum exchange vs an fp32 reference and vs NCCL."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist

from miles_b200.parallel.state import init_parallel_state
from miles_b200.parallel.tensor_parallel import TensorParallel


def main():
    world = int(os.environ["WORLD_SIZE"])
    ps = init_parallel_state()
    dev = ps.device
    H, KL = 2560, 1024
    group = dist.group.WORLD
    tp_f = TensorParallel(group, ps.rank, world, dev, H, 4096, fused=True)
    tp_n = TensorParallel(group, ps.rank, world, dev, H, 4096, fused=False)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    for it, T in enumerate([1000, 4096, 37, 1000, 256]):  # repeated sizes reuse both buffer generations
        g = torch.Generator().manual_seed(100 * it + ps.rank)
        a = (torch.randn(T, KL, generator=g) * 0.5).to(dev).to(torch.bfloat16)
        w = (torch.randn(H, KL, generator=g) * 0.05).to(dev).to(torch.bfloat16)
        res = (torch.randn(T, H, generator=torch.Generator().manual_seed(it)) * 0.5).to(dev).to(torch.bfloat16)
        ref = a.float() @ w.float().t()
        dist.all_reduce(ref)
        ref = ref + res.float()
        y_f = tp_f.linear_allreduce(a, w, residual=res, gemm_status=status)
        y_n = tp_n.linear_allreduce(a, w, residual=res, gemm_status=status)
        tp_f.check_status()
        assert status.item() == 0
        rel = (y_f.float() - ref).abs().max().item() / ref.abs().max().item()
        assert rel < 2e-2, rel
        assert (y_f.float() - y_n.float()).abs().max().item() / ref.abs().max().item() < 2e-2
        # every rank must hold bit-identical sums
        gathered = [torch.empty_like(y_f) for _ in range(world)]
        dist.all_gather(gathered, y_f)
        assert all(torch.equal(gathered[0], t) for t in gathered)
        # MN-major weight (the input-gradient form): a2 [T, H_out_local] @ w2 [H_out_local, H]
        w2 = w.t().contiguous()  # [KL, H]
        y_b = tp_f.linear_allreduce(a, w2, b_mn=True, gemm_status=status)
        ref_b = ref - res.float()
        assert (y_b.float() - ref_b).abs().max().item() / ref_b.abs().max().item() < 2e-2
    if ps.rank == 0:
        print(f"TP_CHECK_OK world={world}")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
