"""Trajectory life-cycle events (attempt start, generation start, attempt end) delivered to registered sinks: a
tracker, a dashboard collector, a test. Sinks never raise into the rollout.

Reference: miles/utils/lifecycle.py (32 lines).
"""
from __future__ import annotations

import time
from typing import Callable

_sinks: list = []


def add_sink(fn: Callable[[dict], None]) -> None:
    _sinks.append(fn)


def clear_sinks() -> None:
    _sinks.clear()


def emit(event: str, sample_index: int, **fields) -> None:
    rec = {"event": event, "sample_index": sample_index, "t": time.time(), **fields}
    for s in list(_sinks):
        try:
            s(rec)
        except Exception:  # noqa: BLE001 - observability must not break generation
            pass


def attempt_start(i: int, **kw) -> None:
    emit("attempt_start", i, **kw)


def gen_start(i: int, **kw) -> None:
    emit("gen_start", i, **kw)


def attempt_end(i: int, **kw) -> None:
    emit("attempt_end", i, **kw)
