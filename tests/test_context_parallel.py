"""Zigzag / contiguous context-parallel layouts: slicing, positions, inverse, tile tables (CPU)."""
import torch

from miles_b200.parallel.context_parallel import (build_cp_tiles, contiguous_bounds, unzigzag, zigzag_bounds,
                                                   zigzag_positions, zigzag_slice)


def test_zigzag_round_trip_and_balance():
    lens = [37, 128, 5, 1000]
    x = torch.arange(sum(lens))[:, None].repeat(1, 3)
    for cp in (1, 2, 4):
        parts = [zigzag_slice(x, lens, cp, r) for r in range(cp)]
        assert sum(p.shape[0] for p in parts) == sum(lens)
        assert torch.equal(unzigzag(parts, lens, cp), x)
        # causal work ~ sum of positions: the zigzag layout keeps it within a few percent across ranks
        work = [float(zigzag_positions(lens, cp, r).float().sum()) for r in range(cp)]
        assert max(work) / max(min(work), 1.0) < 1.1
        for r in range(cp):
            pos = zigzag_positions(lens, cp, r)
            assert pos.numel() == parts[r].shape[0]
    assert zigzag_bounds(8, 2, 0) == [(0, 2), (6, 8)] and zigzag_bounds(8, 2, 1) == [(2, 4), (4, 6)]


def test_cp_tiles_cover_local_rows_with_global_positions():
    lens = [300, 70]
    cp = 2
    for r in range(cp):
        tiles = build_cp_tiles(lens, cp, r)
        local = zigzag_positions(lens, cp, r)
        covered = torch.zeros(local.numel(), dtype=torch.bool)
        for q0, n, kv0, p0 in tiles.tolist():
            assert n <= 128 and not covered[q0:q0 + n].any()
            covered[q0:q0 + n] = True
            assert torch.equal(local[q0:q0 + n], torch.arange(p0, p0 + n, dtype=torch.int32))
            assert kv0 in (0, 300)
        assert covered.all()


def test_contiguous_bounds_pad_to_multiple():
    assert contiguous_bounds(1000, 4, 0, multiple=128) == (0, 256, 1024)
    assert contiguous_bounds(1000, 4, 3, multiple=128) == (768, 1000, 1024)
