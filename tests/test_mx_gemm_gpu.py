"""Block-scaled (MXFP8 / NVFP4) tcgen05 GEMM against an fp32 matmul of the dequantised operands."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, b):
    from miles_b200.ops.mx_gemm import dequantize_operand

    return dequantize_operand(a).float() @ dequantize_operand(b).float().t()


@pytest.mark.parametrize("kind", ["mxfp8", "nvfp4"])
@pytest.mark.parametrize("block_n", [128, 256])
@pytest.mark.parametrize("shape", [(128, 128, 256), (256, 384, 1024), (200, 136, 512), (1024, 2048, 768)])
def test_mx_gemm_dense(kind, shape, block_n):
    from miles_b200.ops.mx_gemm import mx_linear, quantize_operand

    M, N, K = shape
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    x = torch.randn(M, K, device="cuda", generator=g) * torch.rand(M, 1, device="cuda", generator=g) * 3
    w = torch.randn(N, K, device="cuda", generator=g) * 0.05
    a, b = quantize_operand(x, kind), quantize_operand(w, kind)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    y = mx_linear(a, b, status, block_n=block_n).float()
    torch.cuda.synchronize()
    assert int(status) == 0
    ref = _ref(a, b)
    err = (y - ref).abs().max().item()
    assert err <= 2e-2 * ref.abs().max().item() + 1e-3, (kind, shape, err, ref.abs().max().item())
    # and the quantised product is close to the unquantised one (loose: format error, not kernel error)
    full = x.float() @ w.float().t()
    rel = ((y - full).norm() / full.norm()).item()
    assert rel < (0.06 if kind == "mxfp8" else 0.2), (kind, rel)


@pytest.mark.parametrize("block_n", [128, 256])
@pytest.mark.parametrize("kind", ["mxfp8", "nvfp4"])
def test_mx_gemm_scale_selection(kind, block_n):
    """Every K block carries a different power-of-two magnitude, so a wrong scale byte or column shows up at once."""
    from miles_b200.ops.mx_gemm import mx_linear, quantize_operand

    M, N, K = 256, 256, 1024
    blk = 32 if kind == "mxfp8" else 16
    g = torch.Generator(device="cuda").manual_seed(3)
    mag_a = torch.exp2(torch.randint(-6, 6, (M, K // blk), device="cuda", generator=g).float()).repeat_interleave(blk, 1)
    mag_b = torch.exp2(torch.randint(-6, 6, (N, K // blk), device="cuda", generator=g).float()).repeat_interleave(blk, 1)
    x = torch.randn(M, K, device="cuda", generator=g) * mag_a
    w = torch.randn(N, K, device="cuda", generator=g) * mag_b
    a, b = quantize_operand(x, kind), quantize_operand(w, kind)
    y = mx_linear(a, b, block_n=block_n).float()
    ref = _ref(a, b)
    assert (y - ref).abs().max().item() <= 2e-2 * ref.abs().max().item()


@pytest.mark.parametrize("block_n", [128, 256])
@pytest.mark.parametrize("kind", ["mxfp8", "nvfp4"])
def test_mx_gemm_grouped_rows(kind, block_n):
    from miles_b200.ops.mx_gemm import mx_linear, quantize_operand

    G, N, K = 4, 256, 512
    rows = [100, 0, 256, 17]  # rows per group; every group starts on a 128-row boundary
    tiles, off = [], 0
    for gi, r in enumerate(rows):
        for t in range((r + 127) // 128):
            tiles.append([gi, off + 128 * t, min(128, r - 128 * t), 0])
        off += ((r + 127) // 128) * 128
    M = off
    g = torch.Generator(device="cuda").manual_seed(11)
    x = torch.randn(M, K, device="cuda", generator=g)
    w = torch.randn(G * N, K, device="cuda", generator=g) * 0.1
    a, b = quantize_operand(x, kind), quantize_operand(w, kind)
    tg = torch.tensor(tiles + [[0, 0, 0, 0]] * 3, dtype=torch.int32, device="cuda")
    nt = torch.tensor([len(tiles)], dtype=torch.int32, device="cuda")
    y = mx_linear(a, b, tile_group=tg, num_m_tiles=nt, n=N, block_n=block_n).float()
    from miles_b200.ops.mx_gemm import dequantize_operand

    xa, wb = dequantize_operand(a).float(), dequantize_operand(b).float()
    for gi, r0, nr, _ in tiles:
        ref = xa[r0:r0 + nr] @ wb[gi * N:(gi + 1) * N].t()
        assert (y[r0:r0 + nr] - ref).abs().max().item() <= 2e-2 * ref.abs().max().item() + 1e-3, (kind, gi)


@pytest.mark.parametrize("kind", ["mxfp8", "nvfp4"])
@pytest.mark.parametrize("preset", ["qwen3-smoke", "qwen3-smoke-moe"])
def test_model_forward_with_block_scaled_weights(preset, kind):
    """The inference forward with quantised projections / experts stays close to the bf16 forward."""
    from miles_b200.models import ParamStore, build_model, get_config

    cfg = get_config(preset)
    store = ParamStore(cfg, "cuda", torch.bfloat16, init_std=0.05, seed=5)
    model = build_model(cfg, store, "b200")
    g = torch.Generator().manual_seed(1)
    lens = [150, 90]
    T = sum(lens)
    tokens = torch.randint(0, cfg.vocab_size, (T,), generator=g).cuda().int()
    pos = torch.cat([torch.arange(l) for l in lens]).cuda().int()
    cu = torch.tensor([0, 150, 240], dtype=torch.int32, device="cuda")
    rows = torch.arange(0, T - 1).cuda()
    tg = tokens[(rows + 1).long()]
    lp_ref, _ = model.forward_logprobs(tokens, pos, cu, rows, tg, 1.0)
    n = model.enable_block_scaled(kind)
    assert n >= 4 * cfg.num_layers
    calls = {"n": 0}
    orig = model._mx_linear

    def counted(*a, **k):
        calls["n"] += 1
        return orig(*a, **k)

    model._mx_linear = counted
    lp_q, _ = model.forward_logprobs(tokens, pos, cu, rows, tg, 1.0)
    model.check_status()
    assert calls["n"] >= 4 * cfg.num_layers
    assert torch.isfinite(lp_q).all()
    d = (lp_q - lp_ref).abs()
    # format noise only (a wrong operand or scale gives differences of several nats on this random model, whose
    # log-probs spread over ~8 nats): E4M3 keeps ~3 % per element, E2M1 ~12 %
    lim = 0.25 if kind == "mxfp8" else 1.0
    assert d.mean().item() < lim, (preset, kind, d.mean().item(), d.max().item())
    corr = torch.corrcoef(torch.stack([lp_q, lp_ref]))[0, 1].item()
    assert corr > (0.98 if kind == "mxfp8" else 0.85), (preset, kind, corr)
    # a weight update is picked up by refresh
    store.params["layers.0.attn.o.weight"].mul_(0.5)
    model.refresh_block_scaled()
    lp_u, _ = model.forward_logprobs(tokens, pos, cu, rows, tg, 1.0)
    assert (lp_u - lp_q).abs().max().item() > 0
