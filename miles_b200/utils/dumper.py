"""Tensor dumper for train-vs-rollout and baseline-vs-target comparisons.

``Dumper.dump(name, tensor, **tags)`` writes ``<dir>/<phase>/step_<k>/<rank>/<name>.pt``; ``compare_dirs``
walks two dump trees and reports max-abs / relative differences per tensor.  Enabled by
``--dumper-enable --dumper-dir`` (phases ``inference``, ``fwd_only``, ``fwd_bwd``).  Reference:
miles/utils/dumper_utils.py:1-343 and utils/test_utils/comparisons/.
"""
from __future__ import annotations

import os
from typing import Optional

import torch


class Dumper:
    def __init__(self, directory: Optional[str], rank: int = 0, enabled: bool = True):
        self.dir, self.rank, self.enabled = directory, rank, bool(enabled and directory)
        self.phase, self.step = "fwd_only", 0
        self.phases = {"inference", "fwd_only", "fwd_bwd"}

    def configure(self, phase: str, step: int) -> None:
        self.phase, self.step = phase, step

    def dump(self, name: str, tensor: torch.Tensor, **tags) -> None:
        if not self.enabled:
            return
        d = os.path.join(self.dir, self.phase, f"step_{self.step}", f"rank_{self.rank}")
        os.makedirs(d, exist_ok=True)
        torch.save({"tensor": tensor.detach().float().cpu(), "tags": tags}, os.path.join(d, name.replace("/", "_") + ".pt"))


def compare_dirs(a: str, b: str, rtol: float = 1e-2) -> list:
    rows = []
    for root, _, files in os.walk(a):
        for fn in files:
            pa = os.path.join(root, fn)
            pb = os.path.join(b, os.path.relpath(pa, a))
            if not os.path.exists(pb):
                rows.append((os.path.relpath(pa, a), None, None, "missing"))
                continue
            ta, tb = torch.load(pa)["tensor"], torch.load(pb)["tensor"]
            if ta.shape != tb.shape:
                rows.append((os.path.relpath(pa, a), None, None, f"shape {tuple(ta.shape)} vs {tuple(tb.shape)}"))
                continue
            err = (ta - tb).abs().max().item()
            rel = err / (tb.abs().max().item() + 1e-12)
            rows.append((os.path.relpath(pa, a), err, rel, "ok" if rel <= rtol else "DIFF"))
    return rows
