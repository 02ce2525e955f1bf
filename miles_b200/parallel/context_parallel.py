"""Context parallelism: how a packed batch is cut along the sequence and put back together.

Zigzag layout (the default of the reference, needed for a balanced causal load): every sample is split into
``2 * cp`` chunks and rank ``r`` owns chunks ``r`` and ``2 * cp - 1 - r``, so each rank holds an early and a late
piece of every sample. All-gather layout (``--allgather-cp``): the concatenated batch is padded to a multiple of
``cp`` and every rank owns one contiguous piece.

Forward attention under context parallelism gathers K and V over the group (they are ``num_kv_heads / num_q_heads``
of the activation bytes under GQA) and runs the tcgen05 attention kernel on the local queries with tile
descriptors that carry each query chunk's position inside its sequence (``build_cp_tiles``); per-token outputs
(log-probs, entropy, values) are put back in sample order with ``gather_per_token``.

Training under context parallelism (second half of this file): a micro-batch is cut with ``MicroBatch.cp_shard``
(local tokens, the response entries whose logit row is local, whole-sample denominators), K and V are gathered with
a differentiable gather (``gather_kv_autograd``: its backward is the reduce-scatter of dK / dV, written as an
all-reduce so that every backend can run it), per-token losses stay local and the ranks' partial losses add up in
the gradient all-reduce over dp x cp. The PyTorch model path runs this end to end (``attention_zigzag``); on the
sm_100a path the context-parallel attention has a forward kernel path only, so training there runs with cp = 1.

Reference: miles/backends/training_utils/cp_utils.py:19-67,195-303 (zigzag slicing, all_gather_with_cp),
data.py:198-235 (all-gather mode).
"""
from __future__ import annotations

from typing import Sequence

import torch
import torch.distributed as dist


def zigzag_bounds(n: int, cp: int, rank: int) -> list:
    """[(start, end)] of the two chunks of a length-``n`` sample owned by ``rank`` (chunk sizes differ by at most 1)."""
    parts = 2 * cp
    base, rem = divmod(n, parts)
    starts = [i * base + min(i, rem) for i in range(parts + 1)]
    a, b = rank, parts - 1 - rank
    return [(starts[a], starts[a + 1]), (starts[b], starts[b + 1])]


def segments(lens: Sequence[int], cp: int, rank: int, layout: str = "zigzag") -> list:
    """Per sample, the ``(start, end)`` pieces of it that ``rank`` owns. ``zigzag``: an early and a late chunk of every
    sample; ``allgather``: the intersection of the sample with the rank's contiguous piece of the concatenated batch
    (possibly none)."""
    if layout == "zigzag":
        return [zigzag_bounds(n, cp, rank) for n in lens]
    lo, hi, _ = contiguous_bounds(sum(lens), cp, rank)
    out, s0 = [], 0
    for n in lens:
        a, b = max(lo, s0) - s0, min(hi, s0 + n) - s0
        out.append([(a, b)] if b > a else [])
        s0 += n
    return out


def zigzag_slice(x: torch.Tensor, lens: Sequence[int], cp: int, rank: int, layout: str = "zigzag") -> torch.Tensor:
    """Rows of a packed ``[T, ...]`` tensor owned by ``rank`` (samples stay in order, early chunk before late chunk)."""
    if cp == 1:
        return x
    out, s0 = [], 0
    for n, segs in zip(lens, segments(lens, cp, rank, layout)):
        for a, b in segs:
            out.append(x[s0 + a:s0 + b])
        s0 += n
    return torch.cat(out, 0) if out else x[:0]


def zigzag_positions(lens: Sequence[int], cp: int, rank: int, layout: str = "zigzag") -> torch.Tensor:
    """Position of every local token inside its sample (what RoPE and the causal mask need)."""
    out = []
    for segs in segments(lens, cp, rank, layout):
        for a, b in segs:
            out.append(torch.arange(a, b, dtype=torch.int32))
    return torch.cat(out) if out else torch.zeros(0, dtype=torch.int32)


def unzigzag(parts: Sequence[torch.Tensor], lens: Sequence[int], cp: int, layout: str = "zigzag") -> torch.Tensor:
    """Inverse of :func:`zigzag_slice`: ``parts[r]`` are rank ``r``'s rows; returns the packed tensor in sample order."""
    if cp == 1:
        return parts[0]
    cursors = [0] * cp
    segs = [segments(lens, cp, r, layout) for r in range(cp)]
    out = []
    for si in range(len(lens)):
        chunks = []
        for r in range(cp):
            for a, b in segs[r][si]:
                chunks.append((a, parts[r][cursors[r]:cursors[r] + (b - a)]))
                cursors[r] += b - a
        chunks.sort(key=lambda t: t[0])
        out.extend(c for _, c in chunks)
    return torch.cat(out, 0)


def contiguous_bounds(total: int, cp: int, rank: int, multiple: int = 1) -> tuple:
    """All-gather layout: (start, end, padded_total) of the rank's piece of the concatenated batch."""
    unit = cp * multiple
    padded = (total + unit - 1) // unit * unit
    per = padded // cp
    return rank * per, min(total, (rank + 1) * per), padded


def build_cp_tiles(lens: Sequence[int], cp: int, rank: int, tile: int = 128) -> torch.Tensor:
    """Tile table for the attention kernel on a zigzag shard: int32 ``[n, 4]`` rows ``{q_row0, q_rows, kv_row0,
    q_pos0}`` where q rows index the local query tensor and kv rows the gathered (sample-order) K / V."""
    rows, q0, kv0 = [], 0, 0
    for n in lens:
        for a, b in zigzag_bounds(n, cp, rank):
            for c in range(a, b, tile):
                rows.append((q0 + (c - a), min(tile, b - c), kv0, c))
            q0 += b - a
        kv0 += n
    rows.sort(key=lambda r: -(r[3] + r[1]))
    return torch.tensor(rows, dtype=torch.int32).view(-1, 4)


def gather_kv(k_local: torch.Tensor, v_local: torch.Tensor, lens: Sequence[int], cp: int, group) -> tuple:
    """All-gather the zigzag shards of K and V over the group and put them in sample order."""
    if cp == 1:
        return k_local, v_local
    sizes = [sum(b - a for n in lens for a, b in zigzag_bounds(n, cp, r)) for r in range(cp)]
    out = []
    for t in (k_local, v_local):
        parts = [torch.empty((s,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device) for s in sizes]
        dist.all_gather(parts, t.contiguous(), group=group)
        out.append(unzigzag(parts, lens, cp))
    return out[0], out[1]


def gather_per_token(x_local: torch.Tensor, lens: Sequence[int], cp: int, rank: int, group=None) -> torch.Tensor:
    """Per-token values of all ranks in sample order. Each rank scatters its rows into a zero tensor of the full
    length and the group sums them (one all-reduce; differentiable in the reference's sense: every row has exactly
    one non-zero contributor)."""
    if cp == 1:
        return x_local
    total = sum(lens)
    full = torch.zeros((total,) + tuple(x_local.shape[1:]), dtype=x_local.dtype, device=x_local.device)
    s0, cur = 0, 0
    for n in lens:
        for a, b in zigzag_bounds(n, cp, rank):
            full[s0 + a:s0 + b] = x_local[cur:cur + (b - a)]
            cur += b - a
        s0 += n
    if group is not None or dist.is_initialized():
        dist.all_reduce(full, group=group)
    return full


# ---------------------------------------------------------------------------------------------- training under CP
class _GatherRows(torch.autograd.Function):
    """All-gather of per-rank row blocks of different sizes with a gradient: forward scatters the local rows into a
    zero tensor of the total size and sums over the group (any backend can do that), backward sums the gradient of
    the full tensor over the group and keeps the local rows' share (the gradient a reduce-scatter would deliver)."""

    @staticmethod
    def forward(ctx, x, sizes, rank, group):
        ctx.sizes, ctx.rank, ctx.group = sizes, rank, group
        off = sum(sizes[:rank])
        full = x.new_zeros((sum(sizes),) + tuple(x.shape[1:]))
        full[off:off + sizes[rank]] = x
        dist.all_reduce(full, group=group)
        return full

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous().clone()
        dist.all_reduce(g, group=ctx.group)
        off = sum(ctx.sizes[:ctx.rank])
        return g[off:off + ctx.sizes[ctx.rank]], None, None, None


def gather_kv_autograd(k_local: torch.Tensor, v_local: torch.Tensor, lens: Sequence[int], cp: int, rank: int, group,
                       layout: str = "zigzag") -> tuple:
    """K and V of all ranks in sample order, differentiable (see ``_GatherRows``)."""
    sizes = _local_sizes(lens, cp, layout)
    out = []
    for t in (k_local, v_local):
        full = _GatherRows.apply(t, sizes, rank, group)
        parts, off = [], 0
        for s in sizes:
            parts.append(full[off:off + s])
            off += s
        out.append(unzigzag(parts, lens, cp, layout))
    return out[0], out[1]


def attention_zigzag(q_local: torch.Tensor, k_full: torch.Tensor, v_full: torch.Tensor, lens: Sequence[int], cp: int, rank: int,
                     scale: float, layout: str = "zigzag") -> torch.Tensor:
    """Causal attention of the local (zigzag) queries against the gathered keys / values, in plain PyTorch ops
    (autograd path of the PyTorch model; the sm_100a path uses the tile table of ``build_cp_tiles``)."""
    Hq, Hk = q_local.shape[1], k_full.shape[1]
    G = Hq // Hk
    outs, q0, s0 = [], 0, 0
    for n, segs in zip(lens, segments(lens, cp, rank, layout)):
        for a, b in segs:
            if b > a:
                qs = q_local[q0:q0 + (b - a)].transpose(0, 1).float()                        # [Hq, Lq, D]
                ks = k_full[s0:s0 + b].transpose(0, 1).float().repeat_interleave(G, dim=0)   # keys 0 .. b-1 of the sample
                vs = v_full[s0:s0 + b].transpose(0, 1).float().repeat_interleave(G, dim=0)
                att = torch.matmul(qs, ks.transpose(1, 2)) * scale
                qpos = torch.arange(a, b, device=q_local.device)[:, None]
                kpos = torch.arange(0, b, device=q_local.device)[None, :]
                att = att.masked_fill(kpos > qpos, float("-inf"))
                outs.append(torch.matmul(torch.softmax(att, dim=-1), vs).transpose(0, 1).to(q_local.dtype))
            q0 += b - a
        s0 += n
    return torch.cat(outs, 0) if outs else q_local.new_zeros(q_local.shape)


def local_index_map(lens: Sequence[int], cp: int, rank: int, layout: str = "zigzag") -> torch.Tensor:
    """int64 [sum(lens)]: index of every packed token inside the rank's local token list, -1 if another rank owns it."""
    idx = torch.full((sum(lens),), -1, dtype=torch.int64)
    cur, s0 = 0, 0
    for n, segs in zip(lens, segments(lens, cp, rank, layout)):
        for a, b in segs:
            idx[s0 + a:s0 + b] = torch.arange(cur, cur + (b - a))
            cur += b - a
        s0 += n
    return idx


# ---------------------------------------------------------------------------------------------- Ulysses (all-to-all)
class _AllToAllRows(torch.autograd.Function):
    """``all_to_all_single`` over dim 0 with per-peer row counts; the gradient travels the same way back."""

    @staticmethod
    def forward(ctx, x, in_splits, out_splits, group):
        ctx.in_splits, ctx.out_splits, ctx.group = in_splits, out_splits, group
        out = x.new_empty((sum(out_splits),) + tuple(x.shape[1:]))
        dist.all_to_all_single(out, x.contiguous(), out_splits, in_splits, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        gx = g.new_empty((sum(ctx.in_splits),) + tuple(g.shape[1:]))
        dist.all_to_all_single(gx, g.contiguous(), ctx.in_splits, ctx.out_splits, group=ctx.group)
        return gx, None, None, None


def _local_sizes(lens: Sequence[int], cp: int, layout: str = "zigzag") -> list:
    return [sum(b - a for segs in segments(lens, cp, r, layout) for a, b in segs) for r in range(cp)]


def heads_to_sequence(x_local: torch.Tensor, lens: Sequence[int], cp: int, rank: int, group, layout: str = "zigzag") -> torch.Tensor:
    """``[T_local, H, D]`` (this rank's tokens, all heads) -> ``[T, H / cp, D]`` (all tokens in sample order, this
    rank's share of the heads): the first all-to-all of Ulysses-style context parallelism."""
    T, H, D = x_local.shape
    assert H % cp == 0, "the all-to-all layout needs the head count to divide by the context-parallel size"
    sizes = _local_sizes(lens, cp, layout)
    send = x_local.view(T, cp, H // cp, D).transpose(0, 1).reshape(cp * T, H // cp, D)  # block j goes to rank j
    got = _AllToAllRows.apply(send, [T] * cp, sizes, group)
    parts, off = [], 0
    for s in sizes:
        parts.append(got[off:off + s])
        off += s
    return unzigzag(parts, lens, cp, layout)


def sequence_to_heads(y_full: torch.Tensor, lens: Sequence[int], cp: int, rank: int, group, layout: str = "zigzag") -> torch.Tensor:
    """Inverse of :func:`heads_to_sequence` for the attention output."""
    sizes = _local_sizes(lens, cp, layout)
    send = torch.cat([zigzag_slice(y_full, lens, cp, r, layout) for r in range(cp)], 0)  # block r: rank r's tokens, my heads
    T = sizes[rank]
    got = _AllToAllRows.apply(send, sizes, [T] * cp, group)                     # block j: my tokens, rank j's heads
    Hs, D = y_full.shape[1], y_full.shape[2]
    return got.view(cp, T, Hs, D).transpose(0, 1).reshape(T, cp * Hs, D)
