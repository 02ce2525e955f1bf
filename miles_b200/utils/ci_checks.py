"""Self-checks a continuous-integration run turns on with ``--ci-test``.

* per-layer weight hashes, saved next to a checkpoint and compared after loading it (a resumed run must start from
  bit-identical weights);
* the first-step on-policy gate: with the rollout's own weights the first optimizer step of a rollout sees
  ``ppo_kl == 0`` and no clipped token (and a zero KL loss against an identical reference);
* gradient-norm record / replay: one run stores the norm of every step, a later run (other parallel layout, other
  kernels) must reproduce it within 3 %.

Reference counterpart: miles/backends/megatron_utils/ci_utils.py:42-196 and
miles/backends/training_utils/ci_utils.py:12-59.
"""
from __future__ import annotations

import hashlib
import json
import math
import os
import re
from typing import Optional

import torch


def layer_key(name: str) -> str:
    m = re.match(r"layers\.(\d+)\.", name)
    return f"layer{int(m.group(1)):04d}" if m else name.split(".")[0]


def model_hashes_by_layer(store) -> dict:
    """SHA-256 per decoder layer (and per top-level tensor) over name, shape, dtype and raw bytes."""
    hs: dict = {}
    for name in sorted(store.params):
        p = store.params[name]
        h = hs.setdefault(layer_key(name), hashlib.sha256())
        h.update(name.encode())
        h.update(str(tuple(p.shape)).encode())
        h.update(str(p.dtype).encode())
        h.update(p.detach().contiguous().view(torch.uint8).cpu().numpy().tobytes())
    return {k: v.hexdigest() for k, v in sorted(hs.items())}


def hash_file(base_dir: str, iteration: int, ps) -> str:
    d = base_dir if os.path.basename(base_dir.rstrip("/")).startswith("iter_") else os.path.join(base_dir, f"iter_{int(iteration):07d}")
    return os.path.join(d, f"model_hash_tp{ps.tp.rank}_pp{ps.pp.rank}_dp{ps.dp_cp.rank}_ep{ps.ep.rank}.json")


def save_model_hashes(args, store, ps, iteration: int) -> Optional[str]:
    if not (getattr(args, "ci_test", False) and getattr(args, "ci_save_model_hash", False) and getattr(args, "save", None)):
        return None
    path = hash_file(args.save, iteration, ps)
    os.makedirs(os.path.dirname(path), exist_ok=True)
    with open(path, "w") as f:
        json.dump(model_hashes_by_layer(store), f, indent=1, sort_keys=True)
    return path


def check_model_hashes(args, store, ps, iteration: int) -> None:
    if not (getattr(args, "ci_test", False) and getattr(args, "ci_check_model_hash", False) and getattr(args, "load", None)):
        return
    path = hash_file(args.load, iteration, ps)
    if not os.path.isfile(path):
        raise AssertionError(f"weight hash file is missing: {path}")
    want = json.load(open(path))
    have = model_hashes_by_layer(store)
    if want != have:
        bad = sorted(k for k in want.keys() & have.keys() if want[k] != have[k])
        raise AssertionError(f"weights differ from the checkpoint's hashes: mismatched={bad[:5]} "
                             f"missing={sorted(set(want) - set(have))[:5]} extra={sorted(set(have) - set(want))[:5]}")


def check_first_step_kl(args, metrics: dict, step_in_rollout: int, global_step: int) -> None:
    if not getattr(args, "ci_test", False) or getattr(args, "ci_disable_kl_checker", False):
        return
    if step_in_rollout == 0 and "train/ppo_kl" in metrics and "train/pg_clipfrac" in metrics:
        tol = 1e-8 if getattr(args, "lora_rank", 0) else 1e-9
        assert abs(metrics["train/ppo_kl"]) < tol and abs(metrics["train/pg_clipfrac"]) < 1e-10, \
            f"first step of a rollout is not on-policy: {metrics}"
    if global_step == 0 and "train/kl_loss" in metrics and not getattr(args, "use_rollout_routing_replay", False):
        assert abs(metrics["train/kl_loss"]) < 1e-9, f"KL to an identical reference is not zero: {metrics}"


def check_grad_norm(args, grad_norm: float, rollout_id: int, step_id: int, role: str = "actor", rank: int = 0) -> None:
    if rank != 0:
        return
    save, load = getattr(args, "ci_save_grad_norm", None), getattr(args, "ci_load_grad_norm", None)
    if save:
        p = save.format(role=role, rollout_id=rollout_id, step_id=step_id)
        os.makedirs(os.path.dirname(p) or ".", exist_ok=True)
        torch.save(float(grad_norm), p)
    elif load:
        want = float(torch.load(load.format(role=role, rollout_id=rollout_id, step_id=step_id), weights_only=False))
        assert math.isclose(float(grad_norm), want, rel_tol=0.03, abs_tol=0.03), f"gradient norm {grad_norm} != recorded {want}"


def check_rollout_logprobs(args, metrics: dict) -> None:
    """Trainer-vs-rollout log-prob gate of a CI run (reference: training_utils/log_utils.py:262-298): the mean
    absolute difference must stay below 0.03; ``--ci-disable-logprobs-checker`` turns it off."""
    if not getattr(args, "ci_test", False) or getattr(args, "ci_disable_logprobs_checker", False):
        return
    d = metrics.get("train/train_rollout_logprob_abs_diff")
    if d is not None:
        assert d <= 0.03, f"trainer and rollout log-probs differ by {d} on average (limit 0.03)"


def metric_checker_from_args(args):
    """``--ci-metric-checker-key K --ci-metric-checker-threshold X`` (with ``--ci-test``): some evaluation of the run
    must reach ``metrics[K] >= X``; the loop calls ``finalize`` at the end of the run (reference:
    miles/utils/metric_checker.py:6-28)."""
    if getattr(args, "ci_test", False) and getattr(args, "ci_metric_checker_key", None) is not None:
        from .metric_utils import MetricChecker

        thr = args.ci_metric_checker_threshold if args.ci_metric_checker_threshold is not None else 0.0
        return MetricChecker(args.ci_metric_checker_key, float(thr))
    return None


def inject_rollout_data(args, rollout_id: int, generated: list, rep: int, n_rep: int) -> list:
    """``--ci-inject-rollout-data-path`` (CI comparison runs): from ``--ci-inject-rollout-data-start-rollout-id`` on the
    samples just generated are replaced by a recording written with ``--save-debug-rollout-data``, after checking that
    the recording and the generation agree on at least ``--ci-inject-rollout-data-min-match-ratio`` of the response
    tokens (a lower ratio means the engine is not running the weights the recording was made with)."""
    path = getattr(args, "ci_inject_rollout_data_path", None)
    start = getattr(args, "ci_inject_rollout_data_start_rollout_id", None)
    if not path or (start is not None and rollout_id < start):
        return generated
    from .types import Sample

    blob = torch.load(path.format(rollout_id=rollout_id), weights_only=False)
    recorded = [Sample.from_dict(d) for d in blob["samples"]]
    recorded = recorded[rep::n_rep] if n_rep > 1 else recorded
    n = min(len(recorded), len(generated))
    if n:
        ratios = []
        for a, b in zip(recorded[:n], generated[:n]):
            ra, rb = list(a.tokens[-a.response_length:]) if a.response_length else [], \
                list(b.tokens[-b.response_length:]) if b.response_length else []
            m = min(len(ra), len(rb))
            ratios.append(sum(x == y for x, y in zip(ra[:m], rb[:m])) / max(max(len(ra), len(rb)), 1))
        mean = sum(ratios) / len(ratios)
        assert mean >= float(getattr(args, "ci_inject_rollout_data_min_match_ratio", 0.9)), \
            f"generated responses match the recording on {mean:.3f} of the tokens only"
    return recorded
