"""sm_100a kernels vs plain PyTorch fp32 references: GEMM family, norms, rope, swiglu, routing, logprob,
Adam, GAE, quantisers (shape grid with boundary inputs: zeros, max-magnitude, ragged tails)."""
import pytest
import torch

from miles_b200.ops import reference as R
from miles_b200.rl.advantages import vanilla_gae

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rel(got, ref):
    return (got.float() - ref.float()).abs().max().item() / (ref.float().abs().max().item() + 1e-6)


def _each(got, ref, rtol, atol):
    """Every element within ``rtol * |ref| + atol`` (a wrong element inside a large tile cannot hide behind the largest
    magnitude of the tensor)."""
    err = (got.float() - ref.float()).abs()
    bad = err > rtol * ref.float().abs() + atol
    assert not bad.any(), (int(bad.sum()), err[bad].max().item(), ref.float()[bad].abs().min().item())


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (1000, 776, 520), (64, 5120, 2048), (8, 2048, 4096), (300, 151936, 512)])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True)])
def test_gemm_majors_and_tails(ext, M, N, K, a_mn, b_mn):
    if N > 100000 and (a_mn or b_mn):
        pytest.skip("large-N case only for the forward layout")
    torch.manual_seed(0)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    A = torch.randn(M, K, device=DEV, dtype=torch.bfloat16) * 0.5
    B = torch.randn(N, K, device=DEV, dtype=torch.bfloat16) * 0.5
    a = A.t().contiguous() if a_mn else A
    b = B.t().contiguous() if b_mn else B
    ref = A.float() @ B.float().t()
    c = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    ext.gemm(a, b, c, a_mn, b_mn, False, 0, status)
    assert _rel(c, ref) < 1e-2 and status.item() == 0
    rms = ref.pow(2).mean().sqrt().item()
    _each(c, ref, 1.6e-2, 4e-3 * rms)          # bf16 output: two ulps of the element plus accumulation-order noise
    c32 = torch.ones(M, N, device=DEV, dtype=torch.float32)
    ext.gemm(a, b, c32, a_mn, b_mn, True, 0, status)
    assert _rel(c32, ref + 1) < 1e-3
    _each(c32, ref + 1, 1e-3, 1e-3 * rms)      # fp32 accumulate-into output


@pytest.mark.parametrize("T,E,K,align", [(512, 16, 8, 64), (4096, 128, 8, 64), (64, 128, 8, 1), (1, 8, 2, 1)])
def test_moe_permutation_grouped_gemms(ext, T, E, K, align):
    torch.manual_seed(1)
    H, I = 256, 128
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    logits = torch.randn(T, E, device=DEV)
    ids, w, probs = ext.moe_router_topk(logits, None, K, True, True)
    rids, rw, _ = R.router_topk(logits, K, True)
    assert torch.equal(ids.sort(-1).values, rids.to(DEV).sort(-1).values) and torch.allclose(w.sort(-1).values, rw.sort(-1).values, atol=1e-6)
    max_rows = T * K + E * (align - 1)
    counts, offsets, dest, src, tiles, nt = ext.moe_build_permutation(ids, E, max_rows, align)
    live = int(nt[1])
    assert counts.sum().item() == T * K and (offsets[1:] - offsets[:-1] >= counts).all() and int(offsets[-1]) == live
    assert ((offsets[1:] - offsets[:-1]) % align == 0).all()
    # stable order inside each expert and a consistent inverse map
    d = dest.long()
    assert (src[d].long() == torch.arange(T * K, device=DEV)).all()
    flat = ids.reshape(-1).long()
    for e in range(min(E, 4)):
        m = flat == e
        assert (d[m][1:] > d[m][:-1]).all() and (d[m] >= offsets[e]).all() and (d[m] < offsets[e] + counts[e]).all()
    x = torch.randn(T, H, device=DEV, dtype=torch.bfloat16)
    xp = ext.moe_permute(x, src, nt, K)
    valid = src[:live] >= 0
    assert torch.equal(xp[:live][valid], x[(src[:live][valid] // K).long()]) and (xp[:live][~valid] == 0).all()
    W1 = torch.randn(E, I, H, device=DEV, dtype=torch.bfloat16) * 0.05
    y = torch.full((max_rows, I), float("nan"), device=DEV, dtype=torch.bfloat16)
    ext.grouped_gemm_rows(xp, W1, y, tiles, nt, False, False, 0, status)
    exp_of_row = torch.repeat_interleave(torch.arange(E, device=DEV), (offsets[1:] - offsets[:-1]).long())
    ref = torch.einsum("rh,rih->ri", xp[:live].float(), W1[exp_of_row].float())
    assert _rel(y[:live], ref) < 1e-2 and status.item() == 0
    dy = (torch.randn(max_rows, I, device=DEV, dtype=torch.bfloat16) * valid_pad(valid, max_rows)[:, None]).contiguous()
    dx = torch.empty(max_rows, H, device=DEV, dtype=torch.bfloat16)
    ext.grouped_gemm_rows(dy, W1, dx, tiles, nt, True, False, 0, status)
    refdx = torch.einsum("ri,rih->rh", dy[:live].float(), W1[exp_of_row].float())
    assert _rel(dx[:live], refdx) < 1e-2
    if align % 64 == 0:
        dW = torch.zeros(E, I, H, device=DEV, dtype=torch.float32)
        ext.grouped_gemm_contr(dy, xp, dW, offsets, False, 0, status)
        refdW = torch.zeros_like(dW).index_add_(0, exp_of_row, torch.einsum("ri,rh->rih", dy[:live].float(), xp[:live].float()))
        assert _rel(dW, refdW) < 1e-2
    out = ext.moe_combine(y, dest, w, T, K)
    refo = (y[d.view(T, K)].float() * w[..., None]).sum(1)
    assert _rel(out, refo) < 1e-2
    res = torch.randn(T, I, device=DEV, dtype=torch.bfloat16)
    assert _rel(ext.moe_combine(y, dest, w, T, K, res), refo + res.float()) < 1e-2


def valid_pad(valid, n):
    v = torch.zeros(n, device=DEV, dtype=torch.bfloat16)
    v[: valid.numel()] = valid.to(torch.bfloat16)
    return v


def test_norm_rope_swiglu_adam_gae(ext):
    torch.manual_seed(2)
    T, H = 333, 2048
    x = torch.randn(T, H, device=DEV, dtype=torch.bfloat16)
    w = (torch.randn(H, device=DEV) * 0.1 + 1).bfloat16()
    y, rstd = ext.rmsnorm_fwd(x, None, w, 1e-6)
    assert _rel(y, R.rmsnorm(x.float(), w.float(), 1e-6)) < 1e-2
    res = torch.randn_like(x)
    y2, _, h = ext.rmsnorm_fwd(x, res, w, 1e-6)
    assert _rel(h, x.float() + res.float()) < 1e-2 and _rel(y2, R.rmsnorm(h.float(), w.float(), 1e-6)) < 1e-2
    gu = torch.randn(T, 1536, device=DEV, dtype=torch.bfloat16)
    assert _rel(ext.swiglu_fwd(gu), R.swiglu(gu.float())) < 1e-2
    # GAE scan vs the loop
    lens = [1, 31, 32, 33, 200]
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=DEV)
    r, v = torch.randn(sum(lens), device=DEV), torch.randn(sum(lens), device=DEV)
    adv, ret = ext.gae(r, v, cu, 0.99, 0.95)
    for a, b in zip(cu[:-1].tolist(), cu[1:].tolist()):
        ea, er = vanilla_gae(r[a:b][None].double(), v[a:b][None].double(), 0.99, 0.95)
        assert torch.allclose(adv[a:b].double(), ea[0], atol=1e-4) and torch.allclose(ret[a:b].double(), er[0], atol=1e-4)


@pytest.mark.parametrize("rows,cols", [(1, 32), (17, 64), (128, 2048), (300, 4096)])
@pytest.mark.parametrize("kind", ["randn", "zeros", "max", "tiny"])
def test_quantizers_match_reference(ext, rows, cols, kind):
    torch.manual_seed(3)
    x = {"randn": torch.randn(rows, cols) * 3, "zeros": torch.zeros(rows, cols), "max": torch.full((rows, cols), 3.0e38),
         "tiny": torch.randn(rows, cols) * 1e-30}[kind].to(DEV).bfloat16()
    if kind == "max":
        x[0, 0] = -x[0, 0]
    q, e = ext.quant_mxfp8(x)
    rq, re = R.mxfp8_quant(x)
    assert torch.equal(e, re.to(DEV))
    assert torch.equal(q.view(torch.float8_e4m3fn).float(), rq.to(DEV).float())
    assert torch.equal(ext.dequant_mxfp8(q, e).float(), R.mxfp8_dequant(rq, re).to(DEV).bfloat16().float())
    amax = ext.absmax(x)
    assert amax.item() == x.float().abs().max().item()
    if kind != "max":  # fp32 overflow of amax/6*S is saturated differently only at the bf16 maximum
        q4, sf = ext.quant_nvfp4(x, amax)
        code, rsf, gdec = R.nvfp4_quant(x, amax)
        packed = (code[..., 0::2] | (code[..., 1::2] << 4)).to(torch.uint8)
        assert torch.equal(sf.view(torch.float8_e4m3fn).float(), rsf.to(DEV).float())
        mism = (q4 != packed.to(DEV)).float().mean().item()
        assert mism < 2e-3, mism  # ties at rounding boundaries may differ by one code
    if rows % 32 == 0 and cols % 32 == 0:
        yq, s, z = ext.fake_int4_quant(x, 1, 32, True)
        ry, rs, rz = R.fake_int4_quant(x, 1, 32, True)
        assert torch.allclose(s.float(), rs.to(DEV).bfloat16().float(), rtol=1e-2, atol=1e-5)
    qb, sb = ext.quant_fp8_block128(x, False)
    rqb, rsb = R.fp8_block128_quant(x, False)
    assert torch.allclose(sb, rsb.to(DEV), rtol=1e-6, atol=0)
    assert (qb.view(torch.float8_e4m3fn).float() - rqb.to(DEV).float()).abs().max().item() <= 32  # one e4m3 ulp at the top binade


@pytest.mark.parametrize("lens,Hq,Hk", [([128], 4, 4), ([1, 7, 129, 300], 8, 2), ([1000, 24, 513], 4, 1), ([2048, 2048], 32, 4)])
def test_flash_attention_fwd_vs_fp32(ext, lens, Hq, Hk):
    from miles_b200.ops.attention import attention_reference, build_tiles

    torch.manual_seed(3)
    T = sum(lens)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    # q, k, v are slices of one fused projection output, as in the model (row pitch != heads * 128)
    qkv = torch.randn(T, Hq + 2 * Hk, 128, device=DEV, dtype=torch.bfloat16)
    qkv[:, :Hq] *= 2.0  # a wide score range exercises the lazy rescaling of the accumulator
    q, k, v = qkv[:, :Hq], qkv[:, Hq:Hq + Hk], qkv[:, Hq + Hk:]
    tiles = build_tiles(lens).to(DEV)
    scale = 128 ** -0.5
    out, lse = ext.flash_attn_fwd(q, k, v, tiles, scale, status)
    ref, ref_lse = attention_reference(q, k, v, lens, scale)
    assert status.item() == 0
    assert torch.isfinite(out.float()).all()
    assert _rel(out, ref) < 2e-2
    # P travels to the second MMA as bf16: at most 2^-9 * sum p|v| <= 0.002 * max|v| per element, plus the output rounding
    _each(out, ref, 1.6e-2, 5e-3 * v.float().abs().max().item())
    assert (lse - ref_lse).abs().max().item() < 2e-2
    # increasing scores along the sequence force a rescale at every block
    k2 = k.clone()
    ramp = torch.arange(T, device=DEV, dtype=torch.float32)[:, None, None] * 0.05
    q2 = torch.ones_like(q)
    k2 = (torch.ones_like(k).float() * ramp).to(torch.bfloat16)
    out2, lse2 = ext.flash_attn_fwd(q2, k2, v.contiguous(), tiles, scale, status)
    ref2, ref_lse2 = attention_reference(q2, k2, v, lens, scale)
    assert status.item() == 0 and _rel(out2, ref2) < 2e-2 and (lse2 - ref_lse2).abs().max().item() < 5e-2


@pytest.mark.parametrize("T", [1, 3, 8])
def test_small_decode_kernels_vs_fp32(ext, T):
    """Weight-streaming decode kernels (at most 8 rows): fused-norm GEMV, router + pair lists, per-expert up / down."""
    torch.manual_seed(11 + T)
    H, E, K, I, eps = 2048, 128, 8, 768, 1e-6
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    x = torch.randn(T, H, device=DEV, dtype=torch.bfloat16)
    g = (1 + 0.1 * torch.randn(H, device=DEV)).to(torch.bfloat16)
    xn = x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + eps) * g.float()
    # --- projections
    W = torch.randn(5120, H, device=DEV, dtype=torch.bfloat16) * 0.03
    out = torch.empty(T, 5120, device=DEV, dtype=torch.bfloat16)
    ext.small_gemv(x, g, eps, W, None, out, status)
    assert _rel(out, xn @ W.float().t()) < 1e-2
    Wo = torch.randn(H, 4096, device=DEV, dtype=torch.bfloat16) * 0.03
    a = torch.randn(T, 4096, device=DEV, dtype=torch.bfloat16)
    out2 = torch.empty(T, H, device=DEV, dtype=torch.float32)
    ext.small_gemv(a, None, eps, Wo, x, out2, status)
    assert _rel(out2, a.float() @ Wo.float().t() + x.float()) < 2e-3
    # --- router
    Wr = torch.randn(E, H, device=DEV, dtype=torch.bfloat16) * 0.05
    ids = torch.empty(T, K, dtype=torch.int32, device=DEV)
    w = torch.empty(T, K, dtype=torch.float32, device=DEV)
    active = torch.full((1 + E,), -1, dtype=torch.int32, device=DEV)
    pc = torch.empty(E, dtype=torch.int32, device=DEV)
    pl = torch.full((8 * E,), -1, dtype=torch.int32, device=DEV)
    lg = torch.empty(T, E, device=DEV, dtype=torch.float32)
    ext.small_gemv(x, g, eps, Wr, None, lg, status)
    ext.router_small(lg, K, True, ids, w, active, pc, pl)
    logits = xn @ Wr.float().t()
    assert _rel(lg, logits) < 1e-2
    probs = torch.softmax(logits, -1)
    tv, ti = probs.topk(K, -1)
    got_sorted, order = ids.long().sort(-1)
    # near-ties in fp32-vs-bf16 products may swap the last pick: compare the selected probability mass instead
    assert (probs.gather(1, ids.long()).sum(-1) - tv.sum(-1)).abs().max().item() < 2e-3
    ref_w = probs.gather(1, ids.long())
    ref_w = ref_w / ref_w.sum(-1, keepdim=True)
    assert (w - ref_w).abs().max().item() < 1e-2  # bf16 rounding of the normalised input moves the logits a little
    n_act = int(active[0])
    act_e = active[1:1 + n_act].long()
    assert sorted(act_e.tolist()) == sorted(set(ids.flatten().tolist()))
    assert int(pc.sum()) == T * K
    for e in act_e.tolist():
        pairs = pl[8 * e:8 * e + int(pc[e])].long()
        assert (ids.flatten()[pairs] == e).all()
    # --- experts
    W1 = torch.randn(E, 2 * I, H, device=DEV, dtype=torch.bfloat16) * 0.03
    W2 = torch.randn(E, H, I, device=DEV, dtype=torch.bfloat16) * 0.03
    act = torch.zeros(T * K, 2 * I, device=DEV, dtype=torch.bfloat16)
    ext.moe_small_up(x, g, eps, W1, active, pc, pl, min(E, T * K), K, act, status)
    yp = torch.zeros(T * K, H, device=DEV, dtype=torch.bfloat16)
    ext.moe_small_down(act, W2, active, pc, pl, min(E, T * K), yp, status)
    assert status.item() == 0
    flat = ids.flatten().long()
    tok = torch.arange(T * K, device=DEV) // K
    gu = torch.einsum("ph,pnh->pn", xn[tok], W1[flat].float())
    assert _rel(act, gu) < 1e-2
    a = (torch.nn.functional.silu(act[:, :I].float()) * act[:, I:].float()).to(torch.bfloat16)
    ref_y = torch.einsum("pi,phi->ph", a.float(), W2[flat].float())
    assert _rel(yp, ref_y) < 1e-2


@pytest.mark.parametrize("T", [9, 16, 33, 64])
def test_small_gemv_token_groups_vs_fp32(ext, T):
    """Dense projections of decode steps with 9..64 rows: token groups of 8 share the weight fragments."""
    torch.manual_seed(20 + T)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    for N, K in ((5120, 2048), (2048, 4096), (128, 2048)):
        x = torch.randn(T, K, device=DEV, dtype=torch.bfloat16)
        W = torch.randn(N, K, device=DEV, dtype=torch.bfloat16) * 0.03
        res = torch.randn(T, N, device=DEV, dtype=torch.bfloat16)
        ref = x.float() @ W.float().t()
        out = torch.empty(T, N, device=DEV, dtype=torch.bfloat16)
        ext.small_gemv(x, None, 0.0, W, None, out, status)
        assert _rel(out, ref) < 1e-2
        out32 = torch.empty(T, N, device=DEV, dtype=torch.float32)
        ext.small_gemv(x, None, 0.0, W, res, out32, status)
        assert _rel(out32, ref + res.float()) < 2e-3
    assert status.item() == 0


@pytest.mark.parametrize("lens,Hq,Hk", [([128], 4, 4), ([64], 2, 1), ([1, 7, 129, 300], 8, 2), ([1000, 24, 513], 4, 1),
                                        ([2048, 777], 16, 2)])
def test_flash_attention_bwd_vs_fp32(ext, lens, Hq, Hk):
    """dQ / dK / dV of the tcgen05 backward against fp32 autograd of plain attention, element by element."""
    from miles_b200.ops.attention import attention_backward_reference, build_bwd_blocks, build_tiles

    torch.manual_seed(11)
    T = sum(lens)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    q = (torch.randn(T, Hq, 128, device=DEV) * 0.7).bfloat16()
    # k and v as views of one fused buffer (the layout the model hands over): rows have a pitch beyond Hk * 128
    kv = (torch.randn(T, 2 * Hk, 128, device=DEV) * 0.7).bfloat16()
    k, v = kv[:, :Hk], kv[:, Hk:]
    d_o = (torch.randn(T, Hq, 128, device=DEV) * 0.5).bfloat16()
    scale = 128 ** -0.5
    out, lse = ext.flash_attn_fwd(q, k, v, build_tiles(lens).to(DEV), scale, status)
    dq, dk, dv = ext.flash_attn_bwd(q, k, v, out, d_o, lse, build_bwd_blocks(lens).to(DEV), scale, status)
    torch.cuda.synchronize()
    assert status.item() == 0
    rq, rk, rv = attention_backward_reference(q, k, v, d_o, lens, scale)
    for name, got, ref in (("dq", dq, rq), ("dk", dk, rk), ("dv", dv, rv)):
        assert torch.isfinite(got.float()).all(), name
        # bf16 P / dS operands: a few 1e-3 of the gradient's scale per element, never a wrong tile
        tol = 2e-2 * ref.abs().max().item()
        err = (got.float() - ref).abs()
        assert err.max().item() < tol, (name, err.max().item(), tol)
        rel = err.norm().item() / ref.norm().item()
        assert rel < 1e-2, (name, rel)


def test_bounded_peer_wait_expires_and_the_context_stays_usable(ext):
    """A wait on a flag that no peer ever raises must give up after its budget, report it in the status word and
    return, and the next launches must work: two expert-parallel "ranks" are emulated on one device (both map the same
    region), only rank 0 sends, so rank 0's plan kernel waits in vain for rank 1."""
    import time

    R, Bm, H, K, E = 2, 8, 512, 4, 16

    def al(x):
        return (x + 255) // 256 * 256

    off, lay = 0, {}
    for name, nb in (("xg", R * Bm * H * 2), ("ig", R * Bm * K * 4), ("wg", R * Bm * K * 4), ("yb", R * Bm * H * 2),
                     ("fa", R * 8), ("fb", R * 8)):
        lay[name] = off
        off = al(off + nb)

    def fresh():
        region = torch.zeros(off, dtype=torch.uint8, device=DEV)
        layout = [R, Bm, H, K, lay["xg"], lay["ig"], lay["wg"], lay["yb"], lay["fa"], lay["fb"]]
        return region, layout, [region.data_ptr()] * R

    torch.manual_seed(3)
    T = 5
    x = (torch.randn(T, H, device=DEV) * 0.5).bfloat16()
    ln = torch.ones(H, device=DEV, dtype=torch.bfloat16)
    logits = torch.randn(T, E, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ids, w = torch.empty(T, K, dtype=torch.int32, device=DEV), torch.empty(T, K, device=DEV)

    region, layout, bases = fresh()
    ctrl0 = torch.zeros(8, dtype=torch.int64, device=DEV)
    ext.ep_ll_send(x, ln, 1e-6, logits, None, bases, layout, 0, True, ids, w, ctrl0)
    t0 = time.perf_counter()
    src_rows, counts, offsets, dest, row_src, tiles, totals = ext.ep_ll_plan(region.data_ptr(), layout, 0, E, Bm, 1, ctrl0,
                                                                             50_000_000, status)  # 50 ms budget
    torch.cuda.synchronize()
    waited = time.perf_counter() - t0
    assert status.item() == 5, "the expired wait must be reported (5 = a source rank's rows never arrived)"
    assert 0.04 < waited < 2.0, waited
    assert src_rows.tolist() == [T, 0]           # what did arrive is still planned; the silent peer counts as empty
    local = (ids // (E // R)) == 0
    assert int(counts.sum()) == int(local.sum())
    # the context is intact: an ordinary kernel runs, and a complete exchange on fresh buffers works
    status.zero_()
    a = torch.randn(128, 64, device=DEV, dtype=torch.bfloat16)
    c = torch.empty(128, 128, device=DEV, dtype=torch.bfloat16)
    ext.gemm(a, a, c, False, False, False, 0, status)
    torch.cuda.synchronize()
    assert status.item() == 0 and torch.isfinite(c.float()).all()
    region, layout, bases = fresh()
    ctrls = [torch.zeros(8, dtype=torch.int64, device=DEV) for _ in range(R)]
    for me in range(R):
        ext.ep_ll_send(x, ln, 1e-6, logits, None, bases, layout, me, True, ids, w, ctrls[me])
    out = ext.ep_ll_plan(region.data_ptr(), layout, 1, E, Bm, 1, ctrls[1], 50_000_000, status)
    torch.cuda.synchronize()
    assert status.item() == 0 and out[0].tolist() == [T, T]
    assert int(out[1].sum()) == 2 * int(((ids // (E // R)) == 1).sum())   # both sources' picks of rank 1's experts
