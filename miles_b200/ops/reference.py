"""Plain-PyTorch reference implementations of every fused op.

They are the numerical oracle of the GPU tests (run in fp32) and the compute path of the CPU/gloo
configuration.  Shapes and conventions are identical to the CUDA kernels in ``miles_b200/csrc``.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()
    return y.to(x.dtype)


def rope_inv_freq(dim: int, theta: float, scaling: Optional[dict] = None, device=None) -> torch.Tensor:
    """The ``dim / 2`` inverse frequencies of the rotary embedding. ``scaling``: None; ``{"rope_type": "linear",
    "factor"}`` (every frequency divided by the factor); or ``{"rope_type": "llama3", "factor", "low_freq_factor",
    "high_freq_factor", "original_max_position_embeddings"}``: wavelengths beyond ``original / low_freq_factor`` are
    stretched by the factor, those below ``original / high_freq_factor`` are kept, the band between is interpolated
    (the published Llama-3.1 recipe)."""
    import math

    inv = theta ** (-torch.arange(dim // 2, device=device, dtype=torch.float32) / (dim // 2))
    if not scaling:
        return inv
    kind = scaling.get("rope_type") or scaling.get("type")
    factor = float(scaling["factor"])
    if kind == "linear":
        return inv / factor
    assert kind == "llama3", f"rope scaling {kind!r} is not built"
    low, high = float(scaling.get("low_freq_factor", 1.0)), float(scaling.get("high_freq_factor", 4.0))
    orig = float(scaling.get("original_max_position_embeddings", 8192))
    wavelen = 2 * math.pi / inv
    smooth = ((orig / wavelen - low) / (high - low)).clamp(0.0, 1.0)
    mixed = (1 - smooth) * inv / factor + smooth * inv
    return torch.where(wavelen > orig / low, inv / factor, torch.where(wavelen < orig / high, inv, mixed))


def rope_cos_sin(pos: torch.Tensor, dim: int, theta: float, inv_freq: Optional[torch.Tensor] = None):
    inv = inv_freq if inv_freq is not None else theta ** (-torch.arange(dim // 2, device=pos.device, dtype=torch.float32) / (dim // 2))
    ang = pos.float()[:, None] * inv.to(pos.device)[None, :]
    return ang.cos(), ang.sin()


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x: [T, H, D]; rotate-half convention (first half pairs with second half). When ``cos`` covers fewer than D / 2
    frequencies only the first ``2 * cos.shape[-1]`` dimensions of every head are rotated (partial rotary embedding)."""
    if 2 * cos.shape[-1] < x.shape[-1]:
        r = 2 * cos.shape[-1]
        return torch.cat([apply_rope(x[..., :r], cos, sin), x[..., r:]], dim=-1)
    d = x.shape[-1] // 2
    xf = x.float()
    x1, x2 = xf[..., :d], xf[..., d:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).to(x.dtype)


def qk_norm_rope(qkv: torch.Tensor, qw: Optional[torch.Tensor], kw: Optional[torch.Tensor], pos: torch.Tensor,
                 Hq: int, Hk: int, D: int, theta: float, eps: float, inv_freq: Optional[torch.Tensor] = None,
                 rotary_dim: int = 0):
    """qkv [T, (Hq+2Hk)*D] -> q [T,Hq,D], k [T,Hk,D], v [T,Hk,D]. ``inv_freq``: see :func:`rope_inv_freq`;
    ``rotary_dim``: rotate only the first ``rotary_dim`` dimensions of every head (0 = all)."""
    T = qkv.shape[0]
    v3 = qkv.view(T, Hq + 2 * Hk, D)
    q, k, v = v3[:, :Hq], v3[:, Hq:Hq + Hk], v3[:, Hq + Hk:]
    if qw is not None:
        q = rmsnorm(q, qw, eps)
        k = rmsnorm(k, kw, eps)
    cos, sin = rope_cos_sin(pos, rotary_dim or D, theta, inv_freq)
    return apply_rope(q, cos, sin), apply_rope(k, cos, sin), v


def swiglu(gu: torch.Tensor) -> torch.Tensor:
    g, u = gu.float().chunk(2, dim=-1)
    return (F.silu(g) * u).to(gu.dtype)


def attention_varlen(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu: torch.Tensor, scale: float) -> torch.Tensor:
    """Causal attention over packed sequences. q [T,Hq,D], k/v [T,Hk,D], cu int [S+1]."""
    Hq, Hk = q.shape[1], k.shape[1]
    G = Hq // Hk
    out = torch.empty_like(q)
    cu_l = cu.tolist()
    for s in range(len(cu_l) - 1):
        a, b = cu_l[s], cu_l[s + 1]
        if b <= a:
            continue
        qs = q[a:b].transpose(0, 1).float()  # [Hq, L, D]
        ks = k[a:b].transpose(0, 1).float().repeat_interleave(G, dim=0)
        vs = v[a:b].transpose(0, 1).float().repeat_interleave(G, dim=0)
        att = torch.matmul(qs, ks.transpose(1, 2)) * scale
        L = b - a
        mask = torch.ones(L, L, dtype=torch.bool, device=q.device).tril()
        att = att.masked_fill(~mask, float("-inf"))
        o = torch.matmul(torch.softmax(att, dim=-1), vs)
        out[a:b] = o.transpose(0, 1).to(q.dtype)
    return out


def attention_prefix(q: torch.Tensor, k_ctx: torch.Tensor, v_ctx: torch.Tensor, q_start: int, scale: float) -> torch.Tensor:
    """One sequence: queries at absolute positions q_start.. attend causally to the full context k_ctx/v_ctx."""
    Hq, Hk = q.shape[1], k_ctx.shape[1]
    G = Hq // Hk
    Lq, Lk = q.shape[0], k_ctx.shape[0]
    qs = q.transpose(0, 1).float()
    ks = k_ctx.transpose(0, 1).float().repeat_interleave(G, dim=0)
    vs = v_ctx.transpose(0, 1).float().repeat_interleave(G, dim=0)
    att = torch.matmul(qs, ks.transpose(1, 2)) * scale
    qpos = torch.arange(q_start, q_start + Lq, device=q.device)[:, None]
    kpos = torch.arange(Lk, device=q.device)[None, :]
    att = att.masked_fill(kpos > qpos, float("-inf"))
    o = torch.matmul(torch.softmax(att, dim=-1), vs)
    return o.transpose(0, 1).to(q.dtype)


def router_topk(logits: torch.Tensor, K: int, renorm: bool, replay_ids: Optional[torch.Tensor] = None):
    """fp32 logits [T,E] -> ids int32 [T,K], weights fp32 [T,K], probs [T,E]."""
    probs = torch.softmax(logits.float(), dim=-1)
    if replay_ids is not None:
        ids = replay_ids.long().clamp(0, logits.shape[1] - 1)
        w = probs.gather(1, ids)
    else:
        # ties resolve to the lowest expert index, like the kernel
        w, ids = torch.topk(probs, K, dim=-1, sorted=True)
    if renorm:
        w = w / w.sum(-1, keepdim=True).clamp_min(1e-20)
    return ids.to(torch.int32), w, probs


def router_sigmoid_topk(logits: torch.Tensor, K: int, renorm: bool, bias: Optional[torch.Tensor] = None, scaling: float = 1.0,
                        n_group: int = 1, topk_group: int = 1, replay_ids: Optional[torch.Tensor] = None):
    """GLM-4.5 / DeepSeek-V3 routing. fp32 logits [T,E] -> ids int32 [T,K], weights fp32 [T,K], scores [T,E].
    ``scores = sigmoid(logits)``; experts are *chosen* by ``scores + bias`` (inside the ``topk_group`` groups whose two
    best biased scores add up highest, when ``n_group > 1``); the *weights* are the unbiased scores of the chosen experts,
    renormalised to sum to one when ``renorm``, times ``scaling``. Differentiable in ``logits`` through the weights."""
    scores = torch.sigmoid(logits.float())
    if replay_ids is not None:
        ids = replay_ids.long().clamp(0, logits.shape[1] - 1)
    else:
        with torch.no_grad():
            choice = scores + bias.float() if bias is not None else scores.clone()
            if n_group > 1:
                T, E = choice.shape
                grouped = choice.view(T, n_group, E // n_group)
                best = grouped.topk(2, dim=-1)[0].sum(-1)
                keep = torch.zeros_like(best).scatter_(1, best.topk(topk_group, dim=-1)[1], 1.0)
                choice = choice.masked_fill(~keep.bool()[:, :, None].expand_as(grouped).reshape(T, E), 0.0)
            ids = torch.topk(choice, K, dim=-1, sorted=True)[1]
    w = scores.gather(1, ids)
    if renorm:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    return ids.to(torch.int32), w * scaling, scores


def moe_experts(x: torch.Tensor, ids: torch.Tensor, w: torch.Tensor, W1: torch.Tensor, W2: torch.Tensor) -> torch.Tensor:
    """x [T,H]; ids/w [T,K]; W1 [E,2I,H]; W2 [E,H,I] -> [T,H] (dense loop over experts)."""
    T, H = x.shape
    out = torch.zeros(T, H, dtype=torch.float32, device=x.device)
    E = W1.shape[0]
    for e in range(E):
        tok, slot = (ids == e).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        xe = x[tok]
        gu = F.linear(xe, W1[e])
        act = swiglu(gu)
        ye = F.linear(act, W2[e])
        out.index_add_(0, tok, ye.float() * w[tok, slot][:, None].float())
    return out.to(x.dtype)


def logprob_entropy(logits: torch.Tensor, targets: torch.Tensor, inv_temp: float):
    ls = torch.log_softmax(logits.float() * inv_temp, dim=-1)
    lp = ls.gather(-1, targets.long()[:, None])[:, 0]
    ent = -(ls.exp() * ls).sum(-1)
    return lp, ent


def sample(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, generator: Optional[torch.Generator] = None):
    """Row-wise sampling; returns (tokens int64 [B], logprobs fp32 [B]) under the temperature-scaled full softmax."""
    x = logits.float()
    if temperature <= 0:
        tok = x.argmax(-1)
        lp = torch.log_softmax(x, -1).gather(-1, tok[:, None])[:, 0]
        return tok, lp
    x = x / temperature
    full = torch.log_softmax(x, -1)
    filt = x.clone()
    if top_k and 0 < top_k < x.shape[-1]:
        kth = torch.topk(filt, top_k, dim=-1).values[:, -1:]
        filt = filt.masked_fill(filt < kth, float("-inf"))
    if top_p < 1.0:
        sp, si = torch.sort(torch.softmax(filt, -1), dim=-1, descending=True)
        cum = sp.cumsum(-1)
        drop = (cum - sp) >= top_p
        sp = sp.masked_fill(drop, 0.0)
        probs = torch.zeros_like(sp).scatter(-1, si, sp)
    else:
        probs = torch.softmax(filt, -1)
    tok = torch.multinomial(probs, 1, generator=generator)[:, 0]
    return tok, full.gather(-1, tok[:, None])[:, 0]


# ---------------------------------------------------------------- quantisers (oracles for csrc/quant.cu)
_E2M1 = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])


def mxfp8_quant(x: torch.Tensor):
    """1x32 blocks: returns (e4m3 values as float8 tensor, uint8 E8M0 exponents)."""
    cols = x.shape[-1]
    xb = x.float().reshape(-1, cols // 32, 32)
    amax = xb.abs().amax(-1)
    v = amax / 448.0
    e = torch.where(v > 0, torch.ceil(torch.log2(v.clamp_min(1e-45))) + 127, torch.zeros_like(v)).clamp(0, 254)
    scale = torch.where(e > 0, torch.exp2(e - 127), torch.full_like(e, 2.0 ** -127))
    q = (xb / scale[..., None]).clamp(-448, 448).to(torch.float8_e4m3fn)
    return q.reshape(x.shape), e.to(torch.uint8).reshape(*x.shape[:-1], cols // 32)


def mxfp8_dequant(q: torch.Tensor, e: torch.Tensor) -> torch.Tensor:
    cols = q.shape[-1]
    ef = e.float()
    scale = torch.where(ef > 0, torch.exp2(ef - 127), torch.full_like(ef, 2.0 ** -127))
    return (q.float().reshape(-1, cols // 32, 32) * scale.reshape(-1, cols // 32, 1)).reshape(q.shape)


def e2m1_round(a: torch.Tensor) -> torch.Tensor:
    """Round |a| (already scaled) to the E2M1 grid, ties to even code; returns code 0..7."""
    bounds = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], device=a.device)
    # ties: <= at even->(0.25 ->0), (1.25->1.0 code2), (2.5->2 code4), (5.0->4 code6); < at odd boundaries
    le = torch.tensor([True, False, True, False, True, False, True], device=a.device)
    code = torch.zeros_like(a, dtype=torch.int64)
    for b, is_le in zip(bounds.tolist(), le.tolist()):
        code = code + ((a > b) if is_le else (a >= b)).long()
    return code


def nvfp4_quant(x: torch.Tensor, global_amax: Optional[torch.Tensor] = None):
    """1x16 blocks; returns (codes uint8 unpacked [.., cols], block scales float8_e4m3, global decode scale)."""
    cols = x.shape[-1]
    xf = x.float()
    gamax = xf.abs().max() if global_amax is None else global_amax.float().reshape(())
    genc = torch.where(gamax > 0, (448.0 * 6.0) / gamax, torch.ones_like(gamax))
    xb = xf.reshape(-1, cols // 16, 16)
    bamax = xb.abs().amax(-1)
    sf8 = (bamax / 6.0 * genc).clamp(max=448.0).to(torch.float8_e4m3fn)
    sf = sf8.float()
    enc = torch.where(sf > 0, genc / sf, torch.zeros_like(sf))
    scaled = xb * enc[..., None]
    code = e2m1_round(scaled.abs()) + (scaled < 0).long() * 8
    return code.to(torch.uint8).reshape(x.shape), sf8.reshape(*x.shape[:-1], cols // 16), 1.0 / genc


def nvfp4_dequant(code: torch.Tensor, sf8: torch.Tensor, gdec: torch.Tensor) -> torch.Tensor:
    cols = code.shape[-1]
    tbl = _E2M1.to(code.device)
    mag = tbl[(code & 7).long()]
    val = torch.where((code & 8) > 0, -mag, mag)
    return (val.reshape(-1, cols // 16, 16) * sf8.float().reshape(-1, cols // 16, 1) * gdec).reshape(code.shape)


def fp8_block128_quant(x: torch.Tensor, ue8m0: bool = False):
    rows, cols = x.shape
    pr, pc = (-rows) % 128, (-cols) % 128
    xp = F.pad(x.float(), (0, pc, 0, pr))
    xb = xp.reshape((rows + pr) // 128, 128, (cols + pc) // 128, 128).permute(0, 2, 1, 3)
    amax = xb.abs().amax((-1, -2)).clamp_min(1e-10)
    s = amax / 448.0
    if ue8m0:
        s = torch.exp2(torch.ceil(torch.log2(s)))
    q = (xb / s[..., None, None]).clamp(-448, 448)
    q = q.permute(0, 2, 1, 3).reshape(rows + pr, cols + pc)[:rows, :cols].to(torch.float8_e4m3fn)
    return q, s


def fake_int4_quant(x: torch.Tensor, gr: int, gc: int, sym: bool):
    rows, cols = x.shape
    xf = x.float().reshape(rows // gr, gr, cols // gc, gc).permute(0, 2, 1, 3)
    if sym:
        s = (xf.abs().amax((-1, -2)) / 7.0).clamp_min(1e-5)
        z = torch.zeros_like(s)
        q = torch.round(xf / s[..., None, None])
    else:
        mx, mn = xf.amax((-1, -2)), xf.amin((-1, -2))
        s = ((mx - mn) / 15.0).clamp_min(1e-5)
        z = (-torch.round(mn / s)).clamp(0, 15)
        q = torch.round(xf / s[..., None, None]) + z[..., None, None]
    return q.permute(0, 2, 1, 3).reshape(rows, cols), s, z
