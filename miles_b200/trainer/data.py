"""Rollout data -> packed micro-batches on the device.

The rollout side hands the trainer a dict of per-sample lists (key set of the reference's
ray/rollout/train_data_conversion.py:16-47: ``tokens, response_lengths, loss_masks, rewards,
rollout_log_probs, rollout_routed_experts, rollout_mask_sums, ...``).  ``build_micro_batches`` packs
samples into THD micro-batches (no padding) capped by ``max_tokens_per_gpu`` and stages them in pinned
host memory; ``MicroBatch.to_device`` is one asynchronous H2D copy per field.

Response alignment (reference loss_hub/logit_processors.py:11-128): for a sample with prompt length p
and total length n, logits at packed positions ``[p-1, n-1)`` predict tokens ``[p, n)``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Sequence

import torch

from ..utils.seqlen_balancing import balanced_bins, first_fit_pack


@dataclass
class MicroBatch:
    tokens: torch.Tensor          # [T] int32
    positions: torch.Tensor       # [T] int32
    cu_seqlens: torch.Tensor      # [S+1] int32
    max_seqlen: int
    rows: torch.Tensor            # [N] int64 packed row of the logit predicting each response token
    targets: torch.Tensor         # [N] int32
    seg: torch.Tensor             # [N] int64 local sample index of each response token
    resp_cu: torch.Tensor         # [S+1] int64
    loss_mask: torch.Tensor       # [N] float32
    rewards: torch.Tensor         # [S] float32
    denoms: torch.Tensor          # [S] float32 (rollout_mask_sums)
    sample_indices: list          # global sample indices
    rollout_log_probs: Optional[torch.Tensor] = None   # [N]
    teacher_log_probs: Optional[torch.Tensor] = None
    replay: Optional[torch.Tensor] = None              # [T, L_moe, K] int32
    extras: dict = field(default_factory=dict)         # log_probs, ref_log_probs, advantages, returns, values ...
    h2d_bytes: int = 0

    @property
    def num_tokens(self) -> int:
        return int(self.tokens.numel())

    @property
    def num_samples(self) -> int:
        return int(self.cu_seqlens.numel() - 1)

    def cp_shard(self, cp: int, rank: int, layout: str = "zigzag") -> "MicroBatch":
        """This rank's share of the micro-batch under context parallelism (zigzag layout): the local tokens with
        their positions and routing rows, and the response entries whose logit row is local. Per-sample quantities
        (rewards, loss denominators) stay whole, so per-sample means still divide by the sample's full token count
        and the ranks' partial losses add up. ``extras["cp"] = (lens, cp, rank)`` tells the model how to attend."""
        if cp == 1:
            return self
        from ..parallel.context_parallel import local_index_map, segments, zigzag_positions, zigzag_slice

        lens = (self.cu_seqlens[1:] - self.cu_seqlens[:-1]).tolist()
        lmap = local_index_map(lens, cp, rank, layout).to(self.rows.device)
        loc = lmap[self.rows]
        keep = loc >= 0
        f = lambda t: None if t is None else t[keep]
        seg = self.seg[keep]
        counts = torch.zeros(len(lens), dtype=torch.int64, device=seg.device).index_add_(0, seg, torch.ones_like(seg))
        resp_cu = torch.cat([counts.new_zeros(1), counts.cumsum(0)])
        local_lens = [sum(b - a for a, b in segs) for segs in segments(lens, cp, rank, layout)]
        cu = torch.tensor([0] + list(torch.tensor(local_lens).cumsum(0).tolist()), dtype=torch.int32, device=self.cu_seqlens.device)
        mb = MicroBatch(
            tokens=zigzag_slice(self.tokens, lens, cp, rank, layout),
            positions=zigzag_positions(lens, cp, rank, layout).to(self.positions.device),
            cu_seqlens=cu, max_seqlen=max(local_lens) if local_lens else 0, rows=loc[keep], targets=self.targets[keep], seg=seg,
            resp_cu=resp_cu, loss_mask=self.loss_mask[keep], rewards=self.rewards, denoms=self.denoms,
            sample_indices=self.sample_indices, rollout_log_probs=f(self.rollout_log_probs), teacher_log_probs=f(self.teacher_log_probs),
            replay=None if self.replay is None else zigzag_slice(self.replay, lens, cp, rank, layout),
            extras={k: (v[keep] if isinstance(v, torch.Tensor) and v.shape[:1] == keep.shape else v) for k, v in self.extras.items()})
        mb.extras["cp"] = (lens, cp, rank, layout)
        return mb

    def to_device(self, device, non_blocking: bool = True) -> "MicroBatch":
        kw = {}
        nbytes = 0
        for k, v in self.__dict__.items():
            if isinstance(v, torch.Tensor):
                if v.device != torch.device(device):
                    nbytes += v.numel() * v.element_size()
                kw[k] = v.to(device, non_blocking=non_blocking)
            elif k == "extras":
                kw[k] = {a: (b.to(device, non_blocking=non_blocking) if isinstance(b, torch.Tensor) else b) for a, b in v.items()}
            else:
                kw[k] = v
        mb = MicroBatch(**kw)
        mb.h2d_bytes = nbytes
        return mb


def _pin(t: torch.Tensor, pin: bool) -> torch.Tensor:
    return t.pin_memory() if pin else t


def pack_samples(data: dict, idxs: Sequence[int], pin: bool = False, num_moe_layers: int = 0, top_k: int = 0) -> MicroBatch:
    toks, pos, rows, tgts, segs, masks, rlp, tlp, replay = [], [], [], [], [], [], [], [], []
    cu, rcu = [0], [0]
    has_rlp = data.get("rollout_log_probs") is not None
    has_tlp = data.get("teacher_log_probs") is not None
    has_replay = data.get("rollout_routed_experts") is not None and num_moe_layers > 0
    for j, i in enumerate(idxs):
        t = torch.as_tensor(data["tokens"][i], dtype=torch.int32)
        n = int(t.numel())
        r = int(data["response_lengths"][i])
        p = n - r
        assert p >= 1, "a sample needs at least one prompt token"
        toks.append(t)
        pos.append(torch.arange(n, dtype=torch.int32))
        rows.append(torch.arange(cu[-1] + p - 1, cu[-1] + n - 1, dtype=torch.int64))
        tgts.append(t[p:])
        segs.append(torch.full((r,), j, dtype=torch.int64))
        lm = data["loss_masks"][i] if data.get("loss_masks") is not None else None
        masks.append(torch.ones(r, dtype=torch.float32) if lm is None else torch.as_tensor(lm, dtype=torch.float32))
        assert masks[-1].numel() == r, "loss mask must cover exactly the response"
        if has_rlp:
            rlp.append(torch.as_tensor(data["rollout_log_probs"][i], dtype=torch.float32))
        if has_tlp:
            tlp.append(torch.as_tensor(data["teacher_log_probs"][i], dtype=torch.float32))
        if has_replay:
            re = torch.as_tensor(data["rollout_routed_experts"][i], dtype=torch.int32).reshape(-1, num_moe_layers, top_k)
            # the engine reports routing for the n-1 tokens that were fed to the model; the final token of the
            # sample is never an input of a training forward that matters, so pad one row
            if re.shape[0] < n:
                re = torch.cat([re, re[-1:].expand(n - re.shape[0], -1, -1)], 0)
            replay.append(re[:n])
        cu.append(cu[-1] + n)
        rcu.append(rcu[-1] + r)
    sums = data.get("rollout_mask_sums")
    denoms = torch.tensor([float(sums[i]) for i in idxs], dtype=torch.float32) if sums is not None else \
        torch.stack([m.sum() for m in masks])
    mb = MicroBatch(
        tokens=_pin(torch.cat(toks), pin), positions=_pin(torch.cat(pos), pin),
        cu_seqlens=_pin(torch.tensor(cu, dtype=torch.int32), pin), max_seqlen=max(b - a for a, b in zip(cu[:-1], cu[1:])),
        rows=_pin(torch.cat(rows), pin), targets=_pin(torch.cat(tgts), pin), seg=_pin(torch.cat(segs), pin),
        resp_cu=_pin(torch.tensor(rcu, dtype=torch.int64), pin), loss_mask=_pin(torch.cat(masks), pin),
        rewards=_pin(torch.tensor([float(data["rewards"][i]) for i in idxs], dtype=torch.float32), pin),
        denoms=_pin(denoms, pin), sample_indices=list(idxs),
        rollout_log_probs=_pin(torch.cat(rlp), pin) if has_rlp else None,
        teacher_log_probs=_pin(torch.cat(tlp), pin) if has_tlp else None,
        replay=_pin(torch.cat(replay), pin) if has_replay else None,
    )
    return mb


def build_micro_batches(data: dict, *, max_tokens_per_gpu: Optional[int] = None, micro_batch_size: Optional[int] = None,
                        num_micro_batches: Optional[int] = None, pin: bool = False, num_moe_layers: int = 0,
                        top_k: int = 0, sample_ids: Optional[Sequence[int]] = None, weights: str = "tokens",
                        flops_quadratic: float = 1.0 / 12288.0) -> list[MicroBatch]:
    """Dynamic (token-capped, first-fit) or fixed-size micro-batches over the local samples. With
    ``num_micro_batches`` the samples are spread over that many bins by balanced partitioning of their cost:
    token counts, or with ``weights="flops"`` an estimate ``n * (1 + n * flops_quadratic)`` in which the causal
    attention term grows with the square of the length (the default ratio is that of a 2048-wide model with 48
    heads-times-dim per layer; only the relative size of the two terms matters)."""
    ids = list(range(len(data["tokens"]))) if sample_ids is None else list(sample_ids)
    lens = [len(data["tokens"][i]) for i in ids]
    if num_micro_batches is not None:
        cost = lens if weights != "flops" else [int(n * (1.0 + n * flops_quadratic)) + 1 for n in lens]
        bins = balanced_bins(cost, num_micro_batches)
    elif max_tokens_per_gpu:
        bins = first_fit_pack(lens, max_tokens_per_gpu)
    else:
        mbs = micro_batch_size or 1
        bins = [list(range(a, min(a + mbs, len(ids)))) for a in range(0, len(ids), mbs)]
    return [pack_samples(data, [ids[j] for j in b], pin, num_moe_layers, top_k) for b in bins if b]


def num_micro_batches_for(lens: Sequence[int], max_tokens_per_gpu: int) -> int:
    return len(first_fit_pack(lens, max_tokens_per_gpu))


def split_by_dp(data: dict, dp_size: int, balance: bool = False) -> list[list[int]]:
    """Sample indices per DP rank: strided by default, Karmarkar-Karp balanced on request
    (reference: ray/rollout/train_data_conversion.py:274-285)."""
    n = len(data["tokens"])
    if not balance:
        return [list(range(r, n, dp_size)) for r in range(dp_size)]
    from ..utils.seqlen_balancing import karmarkar_karp

    return karmarkar_karp([len(t) for t in data["tokens"]], dp_size, equal_size=(n % dp_size == 0))
