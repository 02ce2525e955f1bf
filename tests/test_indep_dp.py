"""Independent data-parallel cells on CPU (gloo, three processes): cross-cell gradient averaging on a reconfigurable
group, quorum changes between steps (a cell leaves, a healed cell joins and receives an in-memory checkpoint), and
the commit consensus after a host-side failure."""
import socket
from types import SimpleNamespace as NS

import torch
import torch.multiprocessing as mp

from miles_b200.ft.indep_dp import (ReconfigurableGroup, _flatten_state, _unflatten_state, cross_cell_grad_sync,
                                    load_trainer_state, trainer_state)
from miles_b200.models import ParamStore, get_config


def test_state_flattening_sends_shared_storage_once():
    a = torch.arange(6.0)
    state = {"x": a, "y": [a, a.clone()], "n": 3, "d": {"z": a}}
    meta, tensors = _flatten_state(state)
    assert len(tensors) == 2  # `a` once, its clone once
    back = _unflatten_state(meta, [t.clone() for t in tensors])
    assert torch.equal(back["x"], a) and torch.equal(back["d"]["z"], a) and back["n"] == 3 and torch.equal(back["y"][1], a)


def _ports(n):
    out = []
    for _ in range(n):
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            out.append(s.getsockname()[1])
    return out


def _actor(seed):
    cfg = get_config("qwen3-tiny")
    st = ParamStore(cfg, "cpu", torch.float32, seed=seed)
    st.allocate_grads(torch.float32)
    return NS(store=st, opt=None, global_step=0)


def _cell(cell, ports, ret):
    torch.set_num_threads(2)  # several ranks share the host cores
    g = ReconfigurableGroup("gloo", timeout_s=30)
    act = _actor(seed=7)
    # quorum 1: three cells average their gradients
    g.configure("127.0.0.1", ports[0], 1, cell, 3)
    for gr in act.store.grad.values():
        gr.fill_(float(cell + 1))
    loss = torch.tensor([float(cell)])
    assert cross_cell_grad_sync(act, g, loss)
    assert all(torch.allclose(gr, torch.full_like(gr, 2.0)) for gr in act.store.grad.values() if gr.numel())
    assert abs(loss.item() - 1.0) < 1e-6
    if cell == 2:
        g.shutdown()  # this cell leaves between steps (none of its collectives is in flight)
        act = _actor(seed=99)  # ... and comes back later with fresh memory
    else:
        # quorum 2: the two survivors go on, and take a real step so that their state moves
        g.configure("127.0.0.1", ports[1], 2, cell, 2)
        for gr in act.store.grad.values():
            gr.fill_(float(10 * (cell + 1)))
        assert cross_cell_grad_sync(act, g)
        assert all(torch.allclose(gr, torch.full_like(gr, 15.0)) for gr in act.store.grad.values() if gr.numel())
        for t in act.store.flat.values():
            t.add_(0.5)
        act.global_step, act.store.version = 5, 5
    # quorum 3: the healed cell joins; cell 0 streams its state to it
    g.configure("127.0.0.1", ports[2], 3, cell, 3)
    if cell == 0:
        sent = g.send_checkpoint(trainer_state(act), dst=2)
        assert sent > sum(t.numel() * 4 for t in act.store.flat.values())
    elif cell == 2:
        load_trainer_state(act, g.recv_checkpoint(src=0))
        assert act.global_step == 5 and act.store.version == 5
    chk = torch.tensor([sum(float(t.double().sum()) for t in act.store.flat.values())], dtype=torch.float64)
    import torch.distributed as dist

    allc = [torch.zeros_like(chk) for _ in range(3)]
    dist.all_gather(allc, chk, group=g.pg)
    assert allc[0] == allc[1] == allc[2], "cells hold different weights after the transfer"
    # a host-side failure in one cell: nobody commits
    if cell == 1:
        g.report_error(RuntimeError("injected: exception before the all-reduce"))
    for gr in act.store.grad.values():
        gr.fill_(1.0)
    committed = cross_cell_grad_sync(act, g)
    ret[cell] = committed
    g.shutdown()


def test_cells_average_reconfigure_heal_and_agree_on_commit():
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    ports = _ports(3)
    ps = [ctx.Process(target=_cell, args=(c, ports, ret)) for c in range(3)]
    for p in ps:
        p.start()
    for p in ps:
        p.join(180)
        assert p.exitcode == 0
    assert dict(ret) == {0: False, 1: False, 2: False}
