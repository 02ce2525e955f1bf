"""Fused Adam on the GPU against an fp32-master PyTorch Adam.

The case that matters for RL post-training: learning rate 1e-6 on bf16 weights of magnitude ~0.02, where one
update (~1e-6) is a hundred times smaller than half a bf16 ulp (~6e-5). Without an fp32 master the update is
rounded away at every step; with the split master (bf16 weight + 16-bit remainder) it has to accumulate exactly
as it does in a plain fp32 copy."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _ref_adam(w32, grads, lr, b1, b2, eps, wd, scale=1.0):
    """Plain fp32 AdamW (decoupled decay inside the step, the form the kernel implements), one gradient per step."""
    w = w32.clone()
    m = torch.zeros_like(w)
    v = torch.zeros_like(w)
    for t, g in enumerate(grads, 1):
        g = g.float() * scale
        m = b1 * m + (1 - b1) * g
        v = b2 * v + (1 - b2) * g * g
        upd = (m / (1 - b1 ** t)) / ((v / (1 - b2 ** t)).sqrt() + eps)
        w = w - lr * (upd + wd * w)
    return w, m, v


@pytest.mark.parametrize("form", ["split", "fp32_master"])
@pytest.mark.parametrize("g_dtype,mv_dtype", [(torch.float32, torch.float32), (torch.bfloat16, torch.float32),
                                              (torch.bfloat16, torch.bfloat16)])
def test_adam_small_lr_accumulates_like_fp32_master(ext, form, g_dtype, mv_dtype):
    torch.manual_seed(0)
    n, steps, lr = 8 * 4099 + 3, 200, 1e-6  # ragged tail on purpose
    w0 = (torch.randn(n, device=DEV) * 0.02).bfloat16()
    p = w0.clone()
    lo = torch.zeros(n, dtype=torch.int16, device=DEV) if form == "split" else None
    master = w0.float().clone() if form == "fp32_master" else None
    m = torch.zeros(n, dtype=mv_dtype, device=DEV)
    v = torch.zeros(n, dtype=mv_dtype, device=DEV)
    # a persistent drift plus noise: what a real gradient looks like over a few hundred steps
    drift = torch.randn(n, device=DEV)
    grads = [(drift + 0.5 * torch.randn(n, device=DEV)).to(g_dtype) for _ in range(steps)]
    scale = torch.full((1,), 0.5, device=DEV)
    skip = torch.zeros(1, device=DEV)
    for t, g in enumerate(grads, 1):
        ext.adam_step(p, master, g, m, v, lr, 0.9, 0.98, 1e-8, 0.1, t, scale, skip, lo)
    ref_w, ref_m, ref_v = _ref_adam(w0.float(), grads, lr, 0.9, 0.98, 1e-8, 0.1, scale=0.5)
    got = ext.split_master_join(p, lo) if form == "split" else master
    delta, ref_delta = got - w0.float(), ref_w - w0.float()
    assert ref_delta.abs().mean().item() > 5e-5  # the accumulated update is real (and each step was ~1e-6)
    tol = 1e-3 if mv_dtype == torch.float32 else 3e-2  # bf16 moments carry 8 bits
    rel = (delta - ref_delta).norm().item() / ref_delta.norm().item()
    assert rel < tol, rel
    # the bf16 weight is the master rounded to nearest
    assert (p.float() - got).abs().max().item() <= (got.abs().max().item() * 2 ** -8) + 1e-12
    if mv_dtype == torch.float32:
        assert torch.allclose(m, ref_m, rtol=1e-4, atol=1e-7) and torch.allclose(v, ref_v, rtol=1e-4, atol=1e-9)


def test_adam_without_master_loses_the_update(ext):
    """The control: the same run on bare bf16 weights moves almost nothing — the reason the master exists."""
    torch.manual_seed(0)
    n = 8 * 1024
    w0 = (torch.randn(n, device=DEV) * 0.02).bfloat16()
    p = w0.clone()
    m, v = torch.zeros(n, device=DEV), torch.zeros(n, device=DEV)
    g = torch.randn(n, device=DEV)
    for t in range(1, 51):
        ext.adam_step(p, None, g, m, v, 1e-6, 0.9, 0.98, 1e-8, 0.0, t, None, None, None)
    moved = (p != w0).float().mean().item()
    assert moved < 0.05


def test_split_master_roundtrip_and_skip_flag(ext):
    torch.manual_seed(1)
    n = 8 * 777
    w32 = torch.randn(n, device=DEV) * 0.02
    w32[:4] = torch.tensor([0.0, -0.0, 1.0, -3.5e-5], device=DEV)
    p = torch.empty(n, dtype=torch.bfloat16, device=DEV)
    lo = torch.empty(n, dtype=torch.int16, device=DEV)
    ext.split_master_cut(w32, p, lo)
    assert torch.equal(ext.split_master_join(p, lo), w32)  # every fp32 bit comes back
    assert (p.float() - w32).abs().max().item() <= w32.abs().max().item() * 2 ** -8
    # a non-finite gradient norm sets the skip flag: nothing may change
    m, v = torch.zeros(n, device=DEV), torch.zeros(n, device=DEV)
    p0, lo0 = p.clone(), lo.clone()
    ext.adam_step(p, None, torch.randn(n, device=DEV), m, v, 1e-3, 0.9, 0.98, 1e-8, 0.1, 1, torch.ones(1, device=DEV),
                  torch.ones(1, device=DEV), lo)
    assert torch.equal(p, p0) and torch.equal(lo, lo0) and m.abs().sum().item() == 0


def test_flat_adam_streamed_state_equals_resident(ext):
    """FlatAdam with the expert group's state streamed through pinned host memory (partly resident) must produce
    the same bits as the all-resident optimizer (the gradient norm is reduced in a fixed order, so the clip
    coefficient is reproducible too)."""
    from miles_b200.models import ParamStore, get_config
    from miles_b200.trainer.optimizer import FlatAdam, OptimConfig

    cfg = get_config("qwen3-smoke-moe")
    outs = []
    for offload in (False, True):
        store = ParamStore(cfg, torch.device(DEV), torch.bfloat16, seed=5)
        store.allocate_grads(torch.float32, torch.bfloat16)
        oc = OptimConfig(lr=1e-6, master_weights=True, offload_states=offload, offload_resident_frac=0.34,
                         offload_chunk_elems=1 << 16)
        opt = FlatAdam(store, oc)
        g = torch.Generator(device=DEV).manual_seed(9)
        for _ in range(5):
            for t in store.grad.values():
                t.copy_(torch.randn(t.numel(), device=DEV, generator=g).to(t.dtype))
            opt.step(1.0)
        torch.cuda.synchronize()
        outs.append({k: opt.master_fp32(k).clone() for k in store.flat})
        if offload:
            st = opt.state["expert"]
            assert st["offload"] and any(not t.is_cuda for t in st["m"]) and any(t.is_cuda for t in st["m"])
            assert opt.h2d_bytes > 0 and opt.d2h_bytes == opt.h2d_bytes
    for k in outs[0]:
        assert torch.equal(outs[0][k], outs[1][k]), k
