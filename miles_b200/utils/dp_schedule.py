"""Rollout-side schedule of one rollout's training: which samples go to which data-parallel rank, in which
micro-batch, for every optimizer step — computed once, where all sequence lengths are known, so that every rank
walks the same number of micro-batches without agreeing on it at run time.

Rules (reference: miles/utils/dp_schedule.py:31-155):

* the samples of one *rollout* (a rollout may yield several samples: compaction, forks, sub-agents) train in the
  same optimizer step or are dropped together;
* a step takes ``global_batch_size`` rollouts; trailing rollouts form a smaller last step only with
  ``allow_partial_step`` and dynamic batching, and only if they give every rank at least one sample;
* dynamic batching packs a step's samples under ``max_tokens_per_gpu * cp_size`` tokens per micro-batch
  (first-fit decreasing), then splits micro-batches until their count is a multiple of
  ``dp_size * microbatch_group`` (``microbatch_group`` > 1 under interleaved pipeline stages);
  fixed batching cuts chunks of ``micro_batch_size`` samples and requires that multiple;
* micro-batches go to ranks round-robin, or by Karmarkar-Karp on their token counts (``balance``) with the same
  number of micro-batches per rank; with ``workload_fn`` (sequence length -> cost, e.g. forward FLOPs, which grow
  faster than linearly through attention) packing and distribution balance that cost instead of tokens.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Sequence

from .seqlen_balancing import first_fit_pack, karmarkar_karp


@dataclass
class DpSchedule:
    partitions: list = field(default_factory=list)        # per rank: global sample indices, in training order
    micro_batches: list = field(default_factory=list)     # per rank: list of micro-batches = positions into partitions[rank]
    num_microbatches: list = field(default_factory=list)  # per step (same on every rank)
    num_rollouts: list = field(default_factory=list)      # per step

    def for_rank(self, rank: int) -> tuple[list, list]:
        return self.partitions[rank], self.micro_batches[rank]


def _split_to(bins: list, target: int, lengths: Sequence[int]) -> None:
    """Split multi-sample bins (largest token count first) until there are ``target`` bins."""
    while len(bins) < target:
        cand = [b for b in bins if len(b) > 1]
        if not cand:
            break
        b = max(cand, key=lambda x: sum(lengths[i] for i in x))
        bins.remove(b)
        order = sorted(b, key=lambda i: -lengths[i])
        left, right, sl, sr = [], [], 0, 0
        for i in order:  # greedy two-way split by length
            if sl <= sr:
                left.append(i)
                sl += lengths[i]
            else:
                right.append(i)
                sr += lengths[i]
        bins.extend([left, right])


def build_dp_schedule(total_lengths: Sequence[int], rollout_ids: Sequence[int], *, dp_size: int, global_batch_size: int,
                      max_tokens_per_gpu: Optional[int] = None, micro_batch_size: Optional[int] = None, cp_size: int = 1,
                      microbatch_group: int = 1, balance: bool = False, allow_partial_step: bool = False,
                      workload_fn=None) -> DpSchedule:
    dynamic = max_tokens_per_gpu is not None
    if not dynamic and micro_batch_size is None:
        raise ValueError("either max_tokens_per_gpu (dynamic batching) or micro_batch_size is required")
    by_rollout: dict = {}
    for pos, rid in enumerate(rollout_ids):
        by_rollout.setdefault(rid, []).append(pos)
    rids = list(by_rollout)
    full = len(rids) // global_batch_size
    if full < 1:
        raise ValueError(f"{len(rids)} rollouts are fewer than one global batch of {global_batch_size}")
    steps = [global_batch_size] * full
    left = len(rids) - full * global_batch_size
    if left and allow_partial_step and dynamic:
        if sum(len(by_rollout[r]) for r in rids[-left:]) >= dp_size:
            steps.append(left)
    align = dp_size * max(1, microbatch_group)
    out = DpSchedule([[] for _ in range(dp_size)], [[] for _ in range(dp_size)], [], steps)
    start = 0
    for n_roll in steps:
        picked = rids[start:start + n_roll]
        start += n_roll
        samples = [pos for r in picked for pos in by_rollout[r]]
        lens = [total_lengths[i] for i in samples]
        if len(samples) < dp_size:
            raise ValueError(f"a step of {n_roll} rollouts has {len(samples)} samples, fewer than the {dp_size} ranks")
        cost = [float(workload_fn(n)) for n in lens] if workload_fn is not None else None
        if dynamic and cost is not None:
            # cost-balanced packing: as many micro-batches as the token budget asks for, equalised by cost
            n_bins = max(1, -(-sum(lens) // (max_tokens_per_gpu * cp_size)))
            bins = [[i] for i in range(len(lens))] if n_bins >= len(lens) else karmarkar_karp(cost, n_bins, equal_size=False)
            bins = [b for b in bins if b]
            target = max((len(bins) + align - 1) // align * align, align)
            _split_to(bins, target, lens)
            if len(bins) != target:
                raise ValueError(f"{len(samples)} samples cannot fill {target} micro-batches (multiple of {align})")
        elif dynamic:
            bins = first_fit_pack(lens, max_tokens_per_gpu * cp_size, decreasing=True)
            target = max((len(bins) + align - 1) // align * align, align)
            _split_to(bins, target, lens)
            if len(bins) != target:
                raise ValueError(f"{len(samples)} samples cannot fill {target} micro-batches (multiple of {align})")
        else:
            bins = [list(range(i, min(i + micro_batch_size, len(lens)))) for i in range(0, len(lens), micro_batch_size)]
            if len(bins) % align:
                raise ValueError(f"{len(bins)} micro-batches of {micro_batch_size} samples are not a multiple of {align}")
        out.num_microbatches.append(len(bins) // dp_size)
        if balance or cost is not None:
            w = cost if cost is not None else lens
            owner = karmarkar_karp([sum(w[i] for i in b) for b in bins], dp_size, equal_size=True)
        else:
            owner = [list(range(r, len(bins), dp_size)) for r in range(dp_size)]
        for rank, ids in enumerate(owner):
            for k in ids:
                lo = len(out.partitions[rank])
                out.partitions[rank].extend(samples[i] for i in bins[k])
                out.micro_batches[rank].append(list(range(lo, lo + len(bins[k]))))
    return out
