"""Pipeline schedule on CPU (gloo): stage layer ranges, execution order of 1F1B, gradients equal to a single process."""
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from miles_b200.parallel.pipeline_parallel import PipeGroup, PipelineSchedule, stage_layers


def test_stage_layers_cover_the_model():
    for L, P in ((48, 4), (36, 8), (7, 3), (2, 2)):
        spans = [stage_layers(L, P, r) for r in range(P)]
        assert spans[0][0] == 0 and spans[-1][1] == L
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        sizes = [hi - lo for lo, hi in spans]
        assert max(sizes) - min(sizes) <= 1
    assert [stage_layers(10, 3, r, first=2, last=2) for r in range(3)] == [(0, 2), (2, 8), (8, 10)]
    assert stage_layers(5, 1, 0) == (0, 5)
    with pytest.raises(ValueError):
        stage_layers(4, 2, 0, first=3, last=3)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


H, T, M = 16, 6, 5


def _weights(P):
    g = torch.Generator().manual_seed(0)
    return [torch.randn(H, H, generator=g) * 0.3 for _ in range(P)]


def _inputs():
    g = torch.Generator().manual_seed(1)
    return [torch.randn(T + i, H, generator=g) for i in range(M)]  # every micro-batch has its own length


def _worker(rank, world, port, ret):
    torch.set_num_threads(2)  # several ranks share the host cores
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    pg = PipeGroup(None, rank, world, list(range(world)))
    W = _weights(world)[rank].clone().requires_grad_(True)
    xs = _inputs()
    saved = {}

    def meta(mb):
        return (xs[mb].shape, torch.float32)

    def fwd(mb, x_in):
        x = (xs[mb] if x_in is None else x_in).detach().requires_grad_(True)
        with torch.enable_grad():
            y = torch.tanh(x @ W)
        saved[mb] = (x, y)
        return y.detach()

    def bwd(mb, dy):
        x, y = saved.pop(mb)
        if dy is None:
            with torch.enable_grad():
                loss = (y * y).sum()
            loss.backward()
        else:
            y.backward(dy)
        return x.grad

    sch = PipelineSchedule(pg, torch.device("cpu"))
    sch.run_1f1b(M, meta, fwd, bwd)
    assert not saved
    # forward-only pass gives the same last-stage outputs
    outs = {}
    sch2 = PipelineSchedule(pg, torch.device("cpu"))
    sch2.run_forward_only(M, meta, lambda mb, x: outs.setdefault(mb, fwd(mb, x)))
    ret[rank] = (W.grad.clone(), sch.log, outs if rank == world - 1 else None)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_1f1b_matches_single_process(world):
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    Ws = [w.clone().requires_grad_(True) for w in _weights(world)]
    ys = []
    for x in _inputs():
        h = x
        for W in Ws:
            h = torch.tanh(h @ W)
        (h * h).sum().backward()
        ys.append(h.detach())
    for r in range(world):
        grad, log, outs = ret[r]
        assert torch.allclose(grad, Ws[r].grad, atol=1e-5), r
        # 1F1B: at most (stages after this one + 1) micro-batches are in flight, every micro-batch runs F then B once
        inflight = peak = 0
        for kind, mb in log:
            inflight += 1 if kind == "F" else -1
            peak = max(peak, inflight)
        assert peak == min(world - r, M)
        assert sorted(m for k, m in log if k == "F") == list(range(M)) == sorted(m for k, m in log if k == "B")
        if outs is not None:
            for mb in range(M):
                assert torch.allclose(outs[mb], ys[mb], atol=1e-6)
