"""Samples -> the trainer's data dict, and rollout metrics.

Implements the conversions of the reference's miles/ray/rollout/train_data_conversion.py:50-285
(reward post-processing with per-rollout group normalisation, loss-mask defaulting,
``rollout_mask_sums`` so that a trajectory split into several samples counts once) and
miles/ray/rollout/rollout_data_conversion.py:10-51 (trimming the batch to a multiple of the global
batch size), plus the metric definitions of miles/ray/rollout/metrics.py:21-262.
"""
from __future__ import annotations

import math
from collections import defaultdict
from typing import Sequence

from ..rl.rewards import normalize_group_rewards
from ..utils.misc import load_function
from ..utils.types import Sample


def flatten_groups(groups) -> list:
    out = []
    for g in groups:
        if isinstance(g, Sample):
            out.append(g)
        else:
            out.extend(flatten_groups(g))
    return out


def postprocess_rollout_data(args, samples: list) -> list:
    """Drop ``remove_sample`` items and trim to a multiple of the global batch size (unless disabled)."""
    samples = [s for s in samples if not s.remove_sample]
    if getattr(args, "disable_rollout_trim_samples", False) or getattr(args, "use_dynamic_global_batch_size", False):
        return samples
    gbs = getattr(args, "global_batch_size", None)
    if gbs and len(samples) > gbs and len(samples) % gbs:
        samples = samples[: len(samples) // gbs * gbs]
    return samples


def convert_samples_to_train_data(args, samples: Sequence[Sample]) -> dict:
    custom = getattr(args, "custom_convert_samples_to_train_data_path", None)
    if custom:
        return load_function(custom)(args, samples)
    key = getattr(args, "reward_key", None)
    raw = [s.get_reward_value(key) for s in samples]
    post = getattr(args, "custom_reward_post_process_path", None)
    if post:
        raw_r, rewards = load_function(post)(args, samples)
    else:
        raw_r = raw
        rewards = normalize_group_rewards(
            raw, [s.group_index if s.group_index is not None else i for i, s in enumerate(samples)],
            [s.effective_rollout_id if s.effective_rollout_id is not None else i for i, s in enumerate(samples)],
            advantage_estimator=args.advantage_estimator,
            normalize=getattr(args, "rewards_normalization", True) is not False,  # --disable-rewards-normalization
            std_normalization=getattr(args, "grpo_std_normalization", True) and not getattr(args, "disable_grpo_std_normalization", False),
        )
    loss_masks = []
    for s in samples:
        lm = s.loss_mask if s.loss_mask is not None else [1] * s.response_length
        assert len(lm) == s.response_length, f"loss mask length {len(lm)} != response length {s.response_length}"
        if s.remove_sample:
            lm = [0] * s.response_length
        loss_masks.append(lm)
    # trainable-token count of the whole rollout each sample belongs to
    by_rollout: dict = defaultdict(int)
    rid = [(s.group_index, s.effective_rollout_id if s.effective_rollout_id is not None else i) for i, s in enumerate(samples)]
    for r, lm in zip(rid, loss_masks):
        by_rollout[r] += sum(lm)
    data = {
        "tokens": [s.tokens for s in samples],
        "response_lengths": [s.response_length for s in samples],
        "total_lengths": [len(s.tokens) for s in samples],
        "loss_masks": loss_masks,
        "rewards": rewards,
        "raw_reward": raw_r,
        "truncated": [1 if s.status == Sample.Status.TRUNCATED else 0 for s in samples],
        "sample_indices": [s.index for s in samples],
        "rollout_ids": [r[1] for r in rid],
        "rollout_mask_sums": [max(by_rollout[r], 1) for r in rid],
        "weight_versions": [s.weight_versions for s in samples],
        "prompt": [s.prompt for s in samples],
        "metadata": [s.train_metadata for s in samples],
        "num_rollouts": len(set(rid)),
    }
    if all(s.rollout_log_probs is not None for s in samples) and samples:
        data["rollout_log_probs"] = [s.rollout_log_probs for s in samples]
    if all(s.rollout_routed_experts is not None for s in samples) and samples:
        data["rollout_routed_experts"] = [s.rollout_routed_experts for s in samples]
    if all(s.teacher_log_probs is not None for s in samples) and samples:
        data["teacher_log_probs"] = [s.teacher_log_probs for s in samples]
    if all(s.opd_reverse_kl is not None for s in samples) and samples:
        data["opd_reverse_kl"] = [s.opd_reverse_kl for s in samples]
    return data


def _stats(xs: Sequence[float], prefix: str) -> dict:
    if not xs:
        return {}
    n = len(xs)
    mean = sum(xs) / n
    return {f"{prefix}/mean": mean, f"{prefix}/max": max(xs), f"{prefix}/min": min(xs),
            f"{prefix}/std": math.sqrt(sum((x - mean) ** 2 for x in xs) / n)}


def pass_at_k(n: int, c: int, k: int) -> float:
    """Unbiased pass@k estimator from n samples with c correct."""
    if n - c < k:
        return 1.0
    p = 1.0
    for i in range(n - c + 1, n + 1):
        p *= 1.0 - k / i
    return 1.0 - p


def has_repetition(tokens: Sequence[int], min_len: int = 20, times: int = 4) -> bool:
    """True when the tail of the response repeats a block of >= min_len tokens ``times`` times."""
    n = len(tokens)
    for L in range(min_len, n // times + 1):
        block = tokens[n - L:]
        if all(tokens[n - (j + 1) * L:n - j * L] == block for j in range(1, times)):
            return True
    return False


def compute_rollout_metrics(args, samples: Sequence[Sample], rollout_time: float, num_gpus: int = 1) -> dict:
    key = getattr(args, "reward_key", None)
    rewards = [s.get_reward_value(key) for s in samples if s.reward is not None]
    resp = [s.response_length for s in samples]
    m = {}
    m.update({f"rollout/{k}": v for k, v in _stats(rewards, "raw_reward").items()})
    m.update({f"rollout/{k}": v for k, v in _stats(resp, "response_len").items()})
    m["rollout/truncated_ratio"] = sum(s.status == Sample.Status.TRUNCATED for s in samples) / max(len(samples), 1)
    m["rollout/aborted_ratio"] = sum(s.status == Sample.Status.ABORTED for s in samples) / max(len(samples), 1)
    groups: dict = defaultdict(list)
    for s in samples:
        if s.reward is not None:
            groups[s.group_index].append(s.get_reward_value(key))
    if groups:
        zero_std = sum(1 for g in groups.values() if len(g) > 1 and max(g) == min(g))
        m["rollout/zero_std_group_ratio"] = zero_std / len(groups)
        if getattr(args, "log_passrate", False):
            n = max(len(g) for g in groups.values())
            k = 1
            while k <= n:
                m[f"passrate/pass@{k}"] = sum(pass_at_k(len(g), sum(r > 0 for r in g), k) for g in groups.values()) / len(groups)
                k *= 2
    m["rollout/repetition_ratio"] = sum(has_repetition(s.tokens[-s.response_length:]) for s in samples if s.response_length) / max(len(samples), 1)
    m["perf/rollout_time"] = rollout_time
    if rollout_time > 0:
        m["perf/tokens_per_gpu_per_sec"] = sum(resp) / rollout_time / max(num_gpus, 1)
    cat_key = getattr(args, "log_reward_category", None)
    if cat_key:
        # share of samples per value of one field of a dict-valued reward (e.g. an error category)
        cats: dict = defaultdict(int)
        for s in samples:
            if isinstance(s.reward, dict) and cat_key in s.reward:
                cats[s.reward[cat_key]] += 1
        for c, n in cats.items():
            m[f"rollout/error_cat/{c}"] = n / max(len(samples), 1)
    if getattr(args, "log_multi_turn", False):
        # responses of tool / multi-turn rollouts contain observation tokens the model did not write (loss mask 0)
        own = [float(sum(s.loss_mask)) if s.loss_mask is not None else float(s.response_length) for s in samples]
        m.update({f"rollout/{k}": v for k, v in _stats(own, "wo_obs_response_length").items()})
        m["rollout/raw_response_length/clip_ratio"] = sum(r >= args.rollout_max_response_len for r in resp) / max(len(resp), 1)
        rounds = [float((s.metadata or {}).get("round_number", (s.metadata or {}).get("num_turns", 0)) or 0) for s in samples]
        if any(rounds):
            m.update({f"rollout/{k}": v for k, v in _stats(rounds, "multi_turn_metric/round_number").items()})
    if getattr(args, "log_correct_samples", False) and rewards:
        # response-length statistics of the samples that earned the full reward
        ok = [float(s.response_length) for s in samples if s.reward is not None and s.get_reward_value(key) >= 1.0]
        m["rollout/correct_samples/ratio"] = len(ok) / max(len(samples), 1)
        m.update({f"rollout/{k}": v for k, v in _stats(ok, "correct_samples/response_len").items()})
    cached = sum(s.prefix_cache_info.get("cached_tokens", 0) for s in samples)
    total_p = sum(s.prefix_cache_info.get("total_prompt_tokens", 0) for s in samples)
    if total_p:
        m["rollout/prefix_cache_hit_rate"] = cached / total_p
    return m


def rebalance_across_dp(args, data: dict, group, rank: int, size: int) -> dict:
    """``--balance-data``: every data-parallel rank generated its own samples, and their lengths differ; the ranks pool
    what they have and take the partition a common schedule (``utils/dp_schedule.py``) gives them, so that every rank
    trains about the same number of tokens (or, with ``--balance-by-flops``, the same estimated cost) and the same number
    of micro-batches. Rewards and advantages inputs are final per sample at this point, so samples may change ranks freely;
    the samples of one rollout stay in the same optimizer step. Collective over ``group``.
    Reference: the rollout-side schedule of miles/utils/dp_schedule.py:31-155 (one process plans for all ranks there)."""
    import torch.distributed as dist

    from ..utils.dp_schedule import build_dp_schedule

    if size <= 1:
        return data
    gathered = [None] * size
    dist.all_gather_object(gathered, data, group=group)
    list_keys = [k for k, v in data.items() if isinstance(v, list)]
    merged = {k: [x for d in gathered for x in d[k]] for k in list_keys}
    # rollout ids are local to the rank that generated them: make them unique over the pool
    uniq: dict = {}
    merged["rollout_ids"] = [uniq.setdefault((r, rid), len(uniq)) for r, d in enumerate(gathered) for rid in d["rollout_ids"]]
    steps = int(getattr(args, "num_steps_per_rollout", None) or 1)
    n_roll = len(uniq)
    if n_roll < size * steps:
        return data  # too few rollouts to give every rank its share in every step: keep what each rank has
    workload = None
    if getattr(args, "balance_by_flops", False):
        workload = lambda n: float(n) * (1.0 + n / 8192.0)  # noqa: E731 - linear layers plus the quadratic attention term
    dynamic = bool(getattr(args, "use_dynamic_batch_size", False)) and getattr(args, "max_tokens_per_gpu", None)
    try:
        sched = build_dp_schedule(merged["total_lengths"], merged["rollout_ids"], dp_size=size, global_batch_size=n_roll // steps,
                                  max_tokens_per_gpu=args.max_tokens_per_gpu if dynamic else None,
                                  micro_batch_size=None if dynamic else 1, cp_size=int(getattr(args, "context_parallel_size", 1) or 1),
                                  balance=True, allow_partial_step=bool(dynamic), workload_fn=workload)
    except ValueError:
        return data  # the pool does not fit the schedule's divisibility rules: keep the local shares
    mine = sched.partitions[rank]
    out = {k: [merged[k][i] for i in mine] for k in list_keys}
    for k, v in data.items():
        if k not in out:
            out[k] = v
    out["num_rollouts"] = len(set(out["rollout_ids"]))
    out["rebalanced_from"] = {"tokens_before": sum(data["total_lengths"]), "tokens_after": sum(out["total_lengths"])}
    return out
