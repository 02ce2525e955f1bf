"""Out-of-bounds writes: every kernel below writes its output into the middle of a larger buffer whose surroundings hold a
sentinel pattern; after the launch the surroundings must be untouched (and the output fully written: no sentinel left).
Shapes are chosen off the tile sizes so that tail handling is what gets exercised. This is the stand-in for a
bounds-checking tool on kernels whose addressing is hand-written (TMA boxes, vectorised stores, per-expert pair lists)."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"
GUARD = 4096  # elements on each side


class Guarded:
    """A tensor of ``shape`` carved out of a buffer with ``GUARD`` sentinel elements before and after it."""

    def __init__(self, shape, dtype, sentinel):
        n = 1
        for s in shape:
            n *= s
        self.sentinel = sentinel
        self.buf = torch.full((n + 2 * GUARD,), sentinel, dtype=dtype, device=DEV)
        self.t = self.buf[GUARD:GUARD + n].view(shape)
        self.n = n

    def check(self, name, written=True):
        lo, hi = self.buf[:GUARD], self.buf[GUARD + self.n:]
        assert bool((lo == self.sentinel).all()), f"{name}: wrote before its output"
        assert bool((hi == self.sentinel).all()), f"{name}: wrote past its output"
        if written:
            assert not bool((self.t == self.sentinel).any()), f"{name}: left part of its output unwritten"


@pytest.mark.parametrize("M,N,K", [(1, 136, 72), (127, 264, 520), (136, 776, 64), (300, 1000, 136), (513, 8, 256), (520, 264, 72)])
def test_gemm_outputs_stay_inside_their_buffers(ext, M, N, K):
    torch.manual_seed(M)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    A = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    B = torch.randn(N, K, device=DEV, dtype=torch.bfloat16)
    for a_mn, b_mn in ((False, False), (False, True), (True, True)):
        if (a_mn and M % 8) or (b_mn and N % 8):
            continue  # a transposed operand's row pitch (M or N elements) must be a multiple of 16 bytes: refused, not run
        a = A.t().contiguous() if a_mn else A
        b = B.t().contiguous() if b_mn else B
        out = Guarded((M, N), torch.bfloat16, 777.0)
        ext.gemm(a, b, out.t, a_mn, b_mn, False, 0, status)
        torch.cuda.synchronize()
        out.check(f"gemm {M}x{N}x{K} {a_mn}/{b_mn}")
        acc = Guarded((M, N), torch.float32, 12345.0)
        acc.t.zero_()
        ext.gemm(a, b, acc.t, a_mn, b_mn, True, 0, status)
        torch.cuda.synchronize()
        acc.check(f"gemm accumulate {M}x{N}x{K}", written=False)
    assert status.item() == 0


@pytest.mark.parametrize("T,E,K,align", [(33, 16, 4, 64), (257, 8, 2, 1), (1000, 128, 8, 64)])
def test_moe_kernels_stay_inside_their_buffers(ext, T, E, K, align):
    torch.manual_seed(T)
    H, I = 256, 136
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ids, w, _ = ext.moe_router_topk(torch.randn(T, E, device=DEV), None, K, True, True)
    max_rows = T * K + E * (align - 1)
    counts, offsets, dest, src, tiles, nt = ext.moe_build_permutation(ids, E, max_rows, align)
    x = torch.randn(T, H, device=DEV, dtype=torch.bfloat16)
    xp = ext.moe_permute(x, src, nt, K)
    W1 = torch.randn(E, 2 * I, H, device=DEV, dtype=torch.bfloat16) * 0.05
    W2 = torch.randn(E, H, I, device=DEV, dtype=torch.bfloat16) * 0.05
    gu = Guarded((max_rows, 2 * I), torch.bfloat16, 777.0)
    ext.grouped_gemm_rows(xp, W1, gu.t, tiles, nt, False, False, 0, status)
    torch.cuda.synchronize()
    gu.check("grouped gemm (rows)", written=False)  # padding rows between experts are not written
    act = ext.swiglu_fwd(gu.t.contiguous())
    yp = Guarded((max_rows, H), torch.bfloat16, 777.0)
    ext.grouped_gemm_rows(act, W2, yp.t, tiles, nt, False, False, 0, status)
    torch.cuda.synchronize()
    yp.check("grouped gemm (rows, second)", written=False)
    gw = Guarded((E, 2 * I, H), torch.float32, 12345.0)
    gw.t.zero_()
    if align == 64:
        ext.grouped_gemm_contr(gu.t.contiguous(), xp, gw.t, offsets, True, 0, status)
        torch.cuda.synchronize()
        gw.check("grouped gemm (contraction)", written=False)
    assert status.item() == 0


@pytest.mark.parametrize("T", [1, 5, 8, 9, 33, 64])
def test_decode_kernels_stay_inside_their_buffers(ext, T):
    torch.manual_seed(T)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    H, N = 2048, 5120
    x = torch.randn(T, H, device=DEV, dtype=torch.bfloat16)
    g = torch.ones(H, device=DEV, dtype=torch.bfloat16)
    W = torch.randn(N, H, device=DEV, dtype=torch.bfloat16) * 0.03
    out = Guarded((T, N), torch.bfloat16, 777.0)
    ext.small_gemv(x, g if T <= 8 else None, 1e-6, W, None, out.t, status)
    torch.cuda.synchronize()
    out.check(f"small_gemv T={T}")
    # paged decode attention: output rows and the split-KV scratch
    B, Hq, Hk, D, ps = min(T, 8), 8, 2, 128, 64
    lens = [1 + 37 * b for b in range(B)]
    n_pages = 1 + sum((l + ps - 1) // ps for l in lens)
    kc = torch.randn(n_pages * ps, Hk, D, device=DEV, dtype=torch.bfloat16)
    vc = torch.randn(n_pages * ps, Hk, D, device=DEV, dtype=torch.bfloat16)
    bt = torch.zeros(B, 8, dtype=torch.int32, device=DEV)
    nxt = 1
    for b, l in enumerate(lens):
        n = (l + ps - 1) // ps
        bt[b, :n] = torch.arange(nxt, nxt + n, dtype=torch.int32)
        nxt += n
    q = torch.randn(B, Hq, D, device=DEV, dtype=torch.bfloat16)
    sl = torch.tensor(lens, dtype=torch.int32, device=DEV)
    for splits in (1, 5):
        att = Guarded((B, Hq, D), torch.bfloat16, 777.0)
        scratch = Guarded((B * Hq * splits * 130,), torch.float32, 12345.0)
        ext.paged_decode_attention(q, kc, vc, bt, sl, att.t, scratch.t, ps, splits, D ** -0.5)
        torch.cuda.synchronize()
        att.check(f"paged decode attention B={B} splits={splits}")
        scratch.check("paged decode attention scratch", written=False)
    assert status.item() == 0


def test_optimizer_step_stays_inside_its_slices(ext):
    """Adam on a slice of the flat buffers (a weight-decay segment): neighbours on both sides keep their values."""
    torch.manual_seed(0)
    n = 128 * 37
    p = Guarded((n,), torch.bfloat16, 777.0)
    p.t.copy_(torch.randn(n, device=DEV) * 0.02)
    g = torch.randn(n, device=DEV)
    m = Guarded((n,), torch.float32, 12345.0)
    v = Guarded((n,), torch.float32, 12345.0)
    lo = Guarded((n,), torch.int16, 321)
    for t in (m.t, v.t, lo.t):
        t.zero_()
    one, zero = torch.ones(1, device=DEV), torch.zeros(1, device=DEV)
    ext.adam_step(p.t, None, g, m.t, v.t, 1e-3, 0.9, 0.98, 1e-8, 0.1, 1, one, zero, lo.t)
    torch.cuda.synchronize()
    for name, gd in (("param", p), ("m", m), ("v", v), ("lo", lo)):
        gd.check(f"adam_step {name}", written=False)
    assert float(m.t.abs().sum()) > 0
