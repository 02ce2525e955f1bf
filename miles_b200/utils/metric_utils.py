"""Metric helpers: perf derivations (tokens/s, TFLOP/s, MFU), FLOP model, device peak table, CI checker.

Definitions follow the reference: ``perf/actor_train_tok_per_s = tokens / actor_train_time``, MFU =
``3 x forward FLOPs / time / peak`` (miles/utils/train_metric_utils.py:14-60), FLOPs per token from the
model shape (miles/utils/flops_utils.py:69-134), dense bf16 peaks per device
(miles/utils/device_flops.py:6-16).
"""
from __future__ import annotations

from typing import Optional, Sequence

PEAK_BF16_TFLOPS = {"B200": 2250.0, "B300": 2250.0, "GB200": 2500.0, "GB300": 2500.0, "H100": 989.0, "H200": 989.0,
                    "H20": 148.0, "A100": 312.0, "A800": 312.0, "L40S": 362.0, "MI300X": 1307.0}


def device_peak_tflops(name: Optional[str] = None, override: Optional[float] = None) -> float:
    if override:
        return float(override)
    if name is None:
        try:
            import torch

            name = torch.cuda.get_device_name() if torch.cuda.is_available() else ""
        except Exception:
            name = ""
    for k, v in PEAK_BF16_TFLOPS.items():
        if k in name.upper().replace(" ", ""):
            return v
    return 0.0


def forward_flops(cfg, seq_lens: Sequence[int]) -> float:
    """Forward FLOPs of one pass over packed sequences (causal attention counted at half the square)."""
    tokens = float(sum(seq_lens))
    H = cfg.hidden_size
    per_tok = 0.0
    for i in range(cfg.num_layers):
        per_tok += 2 * H * cfg.qkv_dim + 2 * cfg.q_dim * H
        if cfg.layer_is_moe(i):
            per_tok += 2 * H * cfg.num_experts + cfg.moe_top_k * 6 * H * cfg.moe_ffn_hidden_size
        else:
            per_tok += 6 * H * cfg.ffn_hidden_size
    per_tok += 2 * H * cfg.vocab_size
    attn = sum(2 * 2 * cfg.q_dim * (L * L / 2.0) for L in seq_lens) * cfg.num_layers
    return tokens * per_tok + attn


def train_step_flops(cfg, seq_lens: Sequence[int], recompute: bool = True, extra_forwards: int = 1) -> float:
    """Forward + backward (2x) + recomputed forward, plus ``extra_forwards`` log-prob passes (old / reference policy)."""
    return forward_flops(cfg, seq_lens) * (3.0 + (1.0 if recompute else 0.0) + extra_forwards)


def mfu(flops: float, seconds: float, n_gpus: int = 1, peak_tflops: Optional[float] = None) -> float:
    peak = device_peak_tflops(override=peak_tflops)
    if peak <= 0 or seconds <= 0:
        return 0.0
    return flops / seconds / (peak * 1e12 * n_gpus)


def perf_metrics(cfg, seq_lens: Sequence[int], train_time: float, num_gpus: int = 1, log_prob_time: float = 0.0,
                 ref_time: float = 0.0, peak_tflops: Optional[float] = None) -> dict:
    f = forward_flops(cfg, seq_lens)
    out = {}
    if train_time > 0:
        out["perf/actor_train_tflops"] = 3 * f / train_time / 1e12 / num_gpus
        out["perf/actor_train_tok_per_s"] = sum(seq_lens) / train_time
        peak = device_peak_tflops(override=peak_tflops)
        if peak:
            out["perf/actor_train_mfu"] = out["perf/actor_train_tflops"] / peak
    if log_prob_time > 0:
        out["perf/log_probs_tflops"] = f / log_prob_time / 1e12 / num_gpus
    if ref_time > 0:
        out["perf/ref_log_probs_tflops"] = f / ref_time / 1e12 / num_gpus
    return out


class MetricChecker:
    """CI gate on an eval metric: fails the run when the best value never reaches the threshold."""

    def __init__(self, key: str, threshold: float, higher_is_better: bool = True):
        self.key, self.threshold, self.higher = key, threshold, higher_is_better
        self.best: Optional[float] = None

    def update(self, metrics: dict) -> None:
        v = metrics.get(self.key)
        if v is None:
            return
        if self.best is None or (v > self.best if self.higher else v < self.best):
            self.best = float(v)

    def passed(self) -> bool:
        if self.best is None:
            return False
        return self.best >= self.threshold if self.higher else self.best <= self.threshold

    def finalize(self) -> None:
        assert self.passed(), f"metric {self.key} best={self.best} did not reach {self.threshold}"
