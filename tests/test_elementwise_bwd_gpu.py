"""Direct numerics of the fused element-wise kernels' backward passes and of the log-prob / entropy kernel, each
against fp32 PyTorch autograd of the same op (``ops/reference.py``)."""
import pytest
import torch

from miles_b200.ops import reference as R

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def ext():
    from miles_b200.ops import _ext

    return _ext.load(required=True)


def _close(got, want, rtol, atol, frac=1e-3):
    """Element-wise: all but a fraction ``frac`` of the elements within rtol / atol of the fp32 result (bf16 outputs
    round to 3 significant digits), and no element further than 8 times that."""
    got, want = got.float(), want.float()
    err = (got - want).abs()
    tol = atol + rtol * want.abs()
    assert (err > tol).float().mean().item() <= frac, ((err > tol).float().mean().item(), err.max().item())
    assert (err <= 8 * tol).all(), (err / tol).max().item()


@pytest.mark.parametrize("T,H", [(1, 1024), (333, 2048), (700, 5120)])
def test_rmsnorm_backward(ext, T, H):
    torch.manual_seed(T)
    x = torch.randn(T, H, device=DEV).bfloat16()
    w = (torch.randn(H, device=DEV) * 0.1 + 1).bfloat16()
    dy = torch.randn(T, H, device=DEV).bfloat16()
    dres = torch.randn(T, H, device=DEV).bfloat16()
    y, rstd = ext.rmsnorm_fwd(x, None, w, 1e-6)
    xf, wf = x.float().requires_grad_(True), w.float().requires_grad_(True)
    R.rmsnorm(xf, wf, 1e-6).backward(dy.float())
    dw = torch.zeros(H, device=DEV)
    dx = ext.rmsnorm_bwd(dy, x, w, rstd, dres, dw, False)
    _close(dx, xf.grad + dres.float(), 2e-2, 2e-2)
    _close(dw, wf.grad, 2e-2, 2e-2 * max(1.0, T ** 0.5))
    # accumulate into an existing gradient, no residual gradient
    dw2 = torch.ones(H, device=DEV)
    dx2 = ext.rmsnorm_bwd(dy, x, w, rstd, None, dw2, True)
    _close(dx2, xf.grad, 2e-2, 2e-2)
    _close(dw2 - 1.0, wf.grad, 2e-2, 2e-2 * max(1.0, T ** 0.5))


@pytest.mark.parametrize("use_norm", [True, False])
@pytest.mark.parametrize("T,Hq,Hk", [(5, 4, 2), (300, 32, 4), (1000, 16, 8)])
def test_qk_norm_rope_forward_and_backward(ext, T, Hq, Hk, use_norm):
    torch.manual_seed(T + Hq)
    D, theta, eps = 128, 1e6, 1e-6
    qkv = torch.randn(T, (Hq + 2 * Hk) * D, device=DEV).bfloat16()
    pos = torch.randint(0, 9000, (T,), device=DEV, dtype=torch.int32)
    qw = (torch.randn(D, device=DEV) * 0.1 + 1).bfloat16() if use_norm else None
    kw = (torch.randn(D, device=DEV) * 0.1 + 1).bfloat16() if use_norm else None
    q, k, qr, kr = ext.qk_norm_rope_fwd(qkv, qw, kw, pos, Hq, Hk, theta, eps, None, None, None, True)
    qkv_f = qkv.float().requires_grad_(True)
    qwf = qw.float().requires_grad_(True) if use_norm else None
    kwf = kw.float().requires_grad_(True) if use_norm else None
    q_ref, k_ref, v_ref = R.qk_norm_rope(qkv_f, qwf, kwf, pos, Hq, Hk, D, theta, eps)
    _close(q, q_ref, 2e-2, 2e-2)
    _close(k, k_ref, 2e-2, 2e-2)
    dq, dk = torch.randn_like(q), torch.randn_like(k)
    dv = torch.randn(T, Hk, D, device=DEV).bfloat16()
    (q_ref * dq.float()).sum().add((k_ref * dk.float()).sum()).add((v_ref * dv.float()).sum()).backward()
    dqw = torch.zeros(D, device=DEV) if use_norm else None
    dkw = torch.zeros(D, device=DEV) if use_norm else None
    dqkv = ext.qk_norm_rope_bwd(dq, dk, dv, qkv, qw, kw, pos, qr if use_norm else None, kr if use_norm else None, dqw, dkw, Hq, Hk, theta)
    _close(dqkv, qkv_f.grad, 2e-2, 3e-2)
    if use_norm:
        _close(dqw, qwf.grad, 2e-2, 3e-2 * (T * Hq) ** 0.5)
        _close(dkw, kwf.grad, 2e-2, 3e-2 * (T * Hk) ** 0.5)


@pytest.mark.parametrize("scaling", [{"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                                      "original_max_position_embeddings": 8192}, {"rope_type": "linear", "factor": 4.0}])
def test_scaled_rotary_embedding_forward_and_backward(ext, scaling):
    """Llama-3.1 style and linear rope scaling: the kernels read the 64 inverse frequencies from a table."""
    torch.manual_seed(3)
    T, Hq, Hk, D, theta, eps = 257, 8, 2, 128, 5e5, 1e-5
    inv = R.rope_inv_freq(D, theta, scaling, DEV).contiguous()
    assert not torch.allclose(inv, R.rope_inv_freq(D, theta, None, DEV))
    qkv = torch.randn(T, (Hq + 2 * Hk) * D, device=DEV).bfloat16()
    pos = torch.randint(0, 9000, (T,), device=DEV, dtype=torch.int32)
    q, k, _, _ = ext.qk_norm_rope_fwd_scaled(qkv, None, None, pos, Hq, Hk, theta, eps, None, None, None, True, inv, 128)
    qkv_f = qkv.float().requires_grad_(True)
    q_ref, k_ref, v_ref = R.qk_norm_rope(qkv_f, None, None, pos, Hq, Hk, D, theta, eps, inv)
    _close(q, q_ref, 2e-2, 2e-2)
    _close(k, k_ref, 2e-2, 2e-2)
    q_plain, _, _, _ = ext.qk_norm_rope_fwd(qkv, None, None, pos, Hq, Hk, theta, eps, None, None, None, True)
    assert (q.float() - q_plain.float()).abs().max().item() > 0.1, "the table must change the rotation"
    dq, dk = torch.randn_like(q), torch.randn_like(k)
    dv = torch.randn(T, Hk, D, device=DEV).bfloat16()
    (q_ref * dq.float()).sum().add((k_ref * dk.float()).sum()).add((v_ref * dv.float()).sum()).backward()
    dqkv = ext.qk_norm_rope_bwd_scaled(dq, dk, dv, qkv, None, None, pos, None, None, None, None, Hq, Hk, theta, inv, 128)
    _close(dqkv, qkv_f.grad, 2e-2, 3e-2)


@pytest.mark.parametrize("use_norm", [True, False])
def test_partial_rotary_embedding_forward_and_backward(ext, use_norm):
    """Rotary embedding on the first 64 dimensions of every head only (GLM-4.5): d pairs with d + 32, the rest passes."""
    torch.manual_seed(5)
    T, Hq, Hk, D, theta, eps = 301, 8, 2, 128, 1e6, 1e-5
    qkv = torch.randn(T, (Hq + 2 * Hk) * D, device=DEV).bfloat16()
    pos = torch.randint(0, 9000, (T,), device=DEV, dtype=torch.int32)
    qw = (torch.randn(D, device=DEV) * 0.1 + 1).bfloat16() if use_norm else None
    kw = (torch.randn(D, device=DEV) * 0.1 + 1).bfloat16() if use_norm else None
    q, k, qr, kr = ext.qk_norm_rope_fwd_scaled(qkv, qw, kw, pos, Hq, Hk, theta, eps, None, None, None, True, None, 64)
    qkv_f = qkv.float().requires_grad_(True)
    qwf = qw.float().requires_grad_(True) if use_norm else None
    kwf = kw.float().requires_grad_(True) if use_norm else None
    q_ref, k_ref, v_ref = R.qk_norm_rope(qkv_f, qwf, kwf, pos, Hq, Hk, D, theta, eps, None, 64)
    _close(q, q_ref, 2e-2, 2e-2)
    _close(k, k_ref, 2e-2, 2e-2)
    if not use_norm:  # the upper half of every head passes through untouched
        assert torch.equal(q[..., 64:], qkv.view(T, Hq + 2 * Hk, D)[:, :Hq, 64:])
    dq, dk = torch.randn_like(q), torch.randn_like(k)
    dv = torch.randn(T, Hk, D, device=DEV).bfloat16()
    (q_ref * dq.float()).sum().add((k_ref * dk.float()).sum()).add((v_ref * dv.float()).sum()).backward()
    dqw = torch.zeros(D, device=DEV) if use_norm else None
    dkw = torch.zeros(D, device=DEV) if use_norm else None
    dqkv = ext.qk_norm_rope_bwd_scaled(dq, dk, dv, qkv, qw, kw, pos, qr if use_norm else None, kr if use_norm else None, dqw, dkw,
                                       Hq, Hk, theta, None, 64)
    _close(dqkv, qkv_f.grad, 2e-2, 3e-2)
    if use_norm:
        _close(dqw, qwf.grad, 2e-2, 3e-2 * (T * Hq) ** 0.5)
        _close(dkw, kwf.grad, 2e-2, 3e-2 * (T * Hk) ** 0.5)


@pytest.mark.parametrize("T,I", [(1, 768), (333, 768), (257, 9728)])
def test_swiglu_backward(ext, T, I):
    torch.manual_seed(I)
    gu = torch.randn(T, 2 * I, device=DEV).bfloat16()
    dout = torch.randn(T, I, device=DEV).bfloat16()
    guf = gu.float().requires_grad_(True)
    R.swiglu(guf).backward(dout.float())
    _close(ext.swiglu_bwd(dout, gu), guf.grad, 2e-2, 2e-2)
    _close(ext.swiglu_fwd(gu), R.swiglu(gu.float()), 2e-2, 2e-2)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("T,V", [(1, 4096), (77, 151936), (300, 32000)])
def test_logprob_entropy_forward_and_backward(ext, T, V, dtype):
    torch.manual_seed(V % 1000 + T)
    inv_t = 1.0 / 0.8
    logits = (torch.randn(T, V, device=DEV) * 3).to(dtype)
    tg = torch.randint(0, V, (T,), device=DEV, dtype=torch.int32)
    lf = logits.detach().clone().float().requires_grad_(True)   # a leaf of its own (fp32 logits: .float() is no copy)
    lp_ref, ent_ref = R.logprob_entropy(lf, tg, inv_t)
    lp, ent, lse, px = ext.logprob_entropy_fwd(logits, tg, inv_t)
    torch.testing.assert_close(lp, lp_ref.detach(), rtol=1e-4, atol=2e-4)
    torch.testing.assert_close(ent, ent_ref.detach(), rtol=1e-4, atol=2e-4)
    dlp = torch.randn(T, device=DEV)
    dent = torch.randn(T, device=DEV) * 0.1
    (lp_ref * dlp).sum().add((ent_ref * dent).sum()).backward()
    dl = ext.logprob_entropy_bwd(logits.clone(), tg, lse, px, dlp, dent, inv_t)
    assert dl.dtype == torch.bfloat16
    # bf16 output: half a unit in the third significant digit of each element
    _close(dl, lf.grad, 1e-2, 1e-6, frac=2e-3)
    # only the log-prob gradient (no entropy term)
    lf2 = logits.detach().clone().float().requires_grad_(True)
    (R.logprob_entropy(lf2, tg, inv_t)[0] * dlp).sum().backward()
    _close(ext.logprob_entropy_bwd(logits.clone(), tg, lse, px, dlp, None, inv_t), lf2.grad, 1e-2, 1e-6, frac=2e-3)
