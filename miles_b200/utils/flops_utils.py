"""FLOP counts of a training step and model-FLOPs utilisation against a device table.

Reference: miles/utils/flops_utils.py:69-134, miles/utils/device_flops.py:6-16 (B200: 2250 dense bf16 TFLOP/s),
miles/utils/train_metric_utils.py:14-60.
"""
from __future__ import annotations

from typing import Optional, Sequence

DEVICE_BF16_TFLOPS = {"B200": 2250.0, "GB200": 2500.0, "H200": 989.0, "H100": 989.0, "A100": 312.0}


def device_peak_tflops(name: Optional[str] = None) -> float:
    if name is None:
        try:
            import torch

            name = torch.cuda.get_device_name() if torch.cuda.is_available() else ""
        except Exception:  # noqa: BLE001
            name = ""
    for k, v in DEVICE_BF16_TFLOPS.items():
        if k in (name or ""):
            return v
    return 0.0


def forward_flops(cfg, seq_lens: Sequence[int]) -> float:
    """Forward FLOPs of a packed batch: projections and MLP / active experts per token, causal attention per
    sequence (half of the square), LM head per token."""
    T = float(sum(seq_lens))
    H, D = cfg.hidden_size, cfg.head_dim
    per_layer_tok = 2.0 * H * (cfg.q_dim + 2 * cfg.kv_dim) + 2.0 * cfg.q_dim * H
    flops = 0.0
    for i in range(cfg.num_layers):
        if cfg.layer_is_moe(i):
            mlp = cfg.moe_top_k * 3 * 2.0 * H * cfg.moe_ffn_hidden_size + 2.0 * H * cfg.num_experts
        else:
            mlp = 3 * 2.0 * H * cfg.ffn_hidden_size
        flops += T * (per_layer_tok + mlp)
        flops += sum(2 * 2.0 * cfg.num_q_heads * D * (n * (n + 1) / 2.0) for n in seq_lens)
    return flops + T * 2.0 * H * cfg.vocab_size


def train_step_flops(cfg, seq_lens: Sequence[int], recompute: bool = True, extra_forwards: int = 1) -> float:
    """Forward + backward (2x) + recomputed forward, plus ``extra_forwards`` log-prob passes (old / reference policy)."""
    f = forward_flops(cfg, seq_lens)
    return f * (3.0 + (1.0 if recompute else 0.0) + extra_forwards)


def mfu(flops: float, seconds: float, n_gpus: int = 1, peak_tflops: Optional[float] = None) -> float:
    peak = peak_tflops if peak_tflops is not None else device_peak_tflops()
    if peak <= 0 or seconds <= 0:
        return 0.0
    return flops / seconds / (peak * 1e12 * n_gpus)
