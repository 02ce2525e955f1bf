"""Host side of the tcgen05 variable-length causal attention forward.

The kernel works on (128-query tile, head) pairs described by a small int32 table; this module builds the
table from the packed-sequence boundaries and keeps the most recent one, since every layer of a pass uses
the same boundaries.

Reference: the reference selects flash-attn varlen attention for Megatron training
(scripts/run_qwen3_30b_a3b.py:206 ``--attention-backend flash``).
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

TILE_Q = 128


def build_tiles(seq_lens: Sequence[int], prefix_lens: Optional[Sequence[int]] = None,
                kv_starts: Optional[Sequence[int]] = None) -> torch.Tensor:
    """int32 ``[n, 4]`` rows ``{q_row0, q_rows, kv_row0, q_pos0}``, longest key range first.

    ``seq_lens`` are the numbers of query rows per sequence (packed back to back in the q tensor);
    ``prefix_lens`` the numbers of cached positions before the first query of each sequence (keys then
    cover prefix + queries); ``kv_starts`` the first k/v row of each sequence (defaults to the packed
    layout that matches the queries when there is no prefix)."""
    rows = []
    q0 = 0
    kv0 = 0
    for i, n in enumerate(seq_lens):
        n = int(n)
        pre = int(prefix_lens[i]) if prefix_lens is not None else 0
        kvs = int(kv_starts[i]) if kv_starts is not None else kv0
        for c in range(0, n, TILE_Q):
            rows.append((q0 + c, min(TILE_Q, n - c), kvs, pre + c))
        q0 += n
        kv0 += pre + n
    rows.sort(key=lambda r: -(r[3] + r[1]))  # causal work grows with the position: schedule long tiles first
    return torch.tensor(rows, dtype=torch.int32).view(-1, 4)


BLOCK_KV = 128


def build_bwd_blocks(seq_lens: Sequence[int]) -> torch.Tensor:
    """int32 ``[n, 4]`` rows ``{first key row, keys, position of the first key, row one past the sequence}`` for the
    backward kernel (one CTA per 128-key block and KV head), blocks with the most queries after them first."""
    rows = []
    t0 = 0
    for n in seq_lens:
        n = int(n)
        for c in range(0, n, BLOCK_KV):
            rows.append((t0 + c, min(BLOCK_KV, n - c), c, t0 + n))
        t0 += n
    rows.sort(key=lambda r: -(r[3] - r[0]))
    return torch.tensor(rows, dtype=torch.int32).view(-1, 4)


class TileCache:
    """Remembers the tile table of the last ``cu_seqlens`` tensor (identity, not value, is compared)."""

    def __init__(self):
        self._cu = None
        self._tiles = None
        self._bwd_cu = None
        self._bwd = None

    def get_bwd(self, cu: torch.Tensor) -> torch.Tensor:
        if self._bwd_cu is not cu:
            lens = (cu[1:] - cu[:-1]).tolist()
            self._bwd = build_bwd_blocks(lens).to(cu.device, non_blocking=True)
            self._bwd_cu = cu
        return self._bwd

    def get(self, cu: torch.Tensor) -> torch.Tensor:
        if self._cu is not cu:
            lens = (cu[1:] - cu[:-1]).tolist()
            self._tiles = build_tiles(lens).to(cu.device, non_blocking=True)
            self._cu = cu
        return self._tiles


def attention_backward_reference(q, k, v, d_out, seq_lens, scale):
    """fp32 autograd gradients of :func:`attention_reference` (oracle for the backward kernel)."""
    qf, kf, vf = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    out, _ = attention_reference(qf, kf, vf, seq_lens, scale, _keep_graph=True)
    out.backward(d_out.float())
    return qf.grad, kf.grad, vf.grad


def attention_reference(q, k, v, seq_lens, scale, _keep_graph: bool = False):
    """Plain fp32 causal attention over packed sequences (oracle for the tests)."""
    lse = torch.empty(q.shape[1], q.shape[0], dtype=torch.float32, device=q.device)
    g = q.shape[1] // k.shape[1]
    s0 = 0
    outs = []
    for n in seq_lens:
        qs = q[s0:s0 + n].float().transpose(0, 1)                               # [Hq, n, d]
        ks = k[s0:s0 + n].float().transpose(0, 1).repeat_interleave(g, dim=0)
        vs = v[s0:s0 + n].float().transpose(0, 1).repeat_interleave(g, dim=0)
        sc = torch.matmul(qs, ks.transpose(1, 2)) * scale
        mask = torch.ones(n, n, dtype=torch.bool, device=q.device).tril()
        sc = sc.masked_fill(~mask, float("-inf"))
        lse[:, s0:s0 + n] = torch.logsumexp(sc, dim=-1).detach()
        outs.append(torch.matmul(torch.softmax(sc, dim=-1), vs).transpose(0, 1))
        s0 += n
    return torch.cat(outs, 0), lse
