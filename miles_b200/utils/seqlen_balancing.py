"""Sequence-length balancing: Karmarkar-Karp k-way partitioning and first-fit packing.

Used to spread samples over data-parallel ranks with near-equal token counts and to form
micro-batches capped by ``--max-tokens-per-gpu``.  Behaviour matches the helpers in the reference's
miles/utils/seqlen_balancing.py (k-way differencing with an equal-size option, first-fit-decreasing
bins) and the first-fit micro-batch builder of miles/backends/training_utils/data.py:424-537.
"""
from __future__ import annotations

import heapq
from typing import Sequence


def karmarkar_karp(lengths: Sequence[int], k: int, equal_size: bool = False) -> list[list[int]]:
    """Partition indices into k groups minimising the spread of group sums (largest differencing method)."""
    n = len(lengths)
    if k <= 0:
        raise ValueError("k must be positive")
    if equal_size and n % k != 0:
        raise ValueError(f"{n} items cannot be split into {k} equal-size groups")
    order = sorted(range(n), key=lambda i: lengths[i])
    # a state is k sets sorted by sum (descending); heap keyed by -(max - min)
    heap: list = []
    counter = 0

    def push(sets):
        nonlocal counter
        sets = sorted(sets, key=lambda s: -s[0])
        heapq.heappush(heap, (-(sets[0][0] - sets[-1][0]), counter, sets))
        counter += 1

    if equal_size:
        for off in range(0, n, k):
            chunk = order[off:off + k]
            push([(lengths[i], [i]) for i in chunk])
    else:
        for i in order:
            push([(lengths[i], [i])] + [(0, []) for _ in range(k - 1)])
    if not heap:
        return [[] for _ in range(k)]
    while len(heap) > 1:
        _, _, a = heapq.heappop(heap)
        _, _, b = heapq.heappop(heap)
        merged = [(a[i][0] + b[k - 1 - i][0], a[i][1] + b[k - 1 - i][1]) for i in range(k)]
        push(merged)
    _, _, final = heap[0]
    parts = [sorted(s[1]) for s in final]
    parts.sort(key=lambda p: (p[0] if p else n))
    return parts


def first_fit_pack(lengths: Sequence[int], capacity: int, decreasing: bool = False) -> list[list[int]]:
    """Greedy first-fit bins of total length <= capacity (an over-long item gets a bin of its own)."""
    idx = list(range(len(lengths)))
    if decreasing:
        idx.sort(key=lambda i: -lengths[i])
    bins: list[list[int]] = []
    sums: list[int] = []
    for i in idx:
        placed = False
        for b in range(len(bins)):
            if sums[b] + lengths[i] <= capacity:
                bins[b].append(i)
                sums[b] += lengths[i]
                placed = True
                break
        if not placed:
            bins.append([i])
            sums.append(lengths[i])
    return bins


def balanced_bins(lengths: Sequence[int], num_bins: int) -> list[list[int]]:
    """Exactly ``num_bins`` bins with balanced sums (used when all DP ranks must run the same number of micro-batches)."""
    num_bins = max(1, min(num_bins, max(1, len(lengths))))
    parts = karmarkar_karp(lengths, num_bins)
    return [p for p in parts]
