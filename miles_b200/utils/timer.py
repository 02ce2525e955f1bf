"""Phase timers (``perf/<name>_time``).

A process-wide ``Timer`` keyed by name with a ``@timer`` decorator / context manager and an
``inverse_timer`` that carves a wait out of an enclosing span, as in the reference's
miles/utils/timer.py:15-99.  Host spans use ``time.perf_counter``; device spans can be recorded with CUDA
events through ``cuda_span`` so that a phase is timed on the stream it runs on.
"""
from __future__ import annotations

import functools
import time
from contextlib import contextmanager
from typing import Callable, Optional


class Timer:
    _instance: Optional["Timer"] = None

    def __new__(cls):
        if cls._instance is None:
            cls._instance = super().__new__(cls)
            cls._instance.timers = {}
            cls._instance.start_time = {}
            cls._instance.sinks = []
            cls._instance.cuda_spans = []
        return cls._instance

    def add_sink(self, fn: Callable[[str, float, float], None]) -> None:
        self.sinks.append(fn)

    def start(self, name: str) -> None:
        assert name not in self.start_time, f"timer {name} already started"
        self.start_time[name] = time.perf_counter()

    def end(self, name: str) -> float:
        assert name in self.start_time, f"timer {name} was not started"
        t0 = self.start_time.pop(name)
        t1 = time.perf_counter()
        self.add(name, t1 - t0)
        for s in self.sinks:
            s(name, t0, t1)
        return t1 - t0

    def add(self, name: str, seconds: float) -> None:
        self.timers[name] = self.timers.get(name, 0.0) + seconds

    def reset(self, name: Optional[str] = None) -> None:
        if name is None:
            self.timers = {}
        else:
            self.timers.pop(name, None)

    def log_dict(self) -> dict:
        self.flush_cuda()
        return dict(self.timers)

    @contextmanager
    def context(self, name: str):
        self.start(name)
        try:
            yield
        finally:
            self.end(name)

    @contextmanager
    def cuda_span(self, name: str):
        """Time a span on the current CUDA stream with events (resolved lazily, no sync here)."""
        import torch

        if not torch.cuda.is_available():
            with self.context(name):
                yield
            return
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        try:
            yield
        finally:
            b.record()
            self.cuda_spans.append((name, a, b))

    def flush_cuda(self) -> None:
        if not self.cuda_spans:
            return
        import torch

        torch.cuda.synchronize()
        for name, a, b in self.cuda_spans:
            self.add(name, a.elapsed_time(b) / 1e3)
        self.cuda_spans = []


def timer(name_or_func=None):
    """``@timer`` / ``@timer("name")`` decorator, or ``with timer("name"):`` context manager."""
    if isinstance(name_or_func, str) or name_or_func is None:
        name = name_or_func

        class _Ctx:
            def __enter__(self_inner):
                Timer().start(name)

            def __exit__(self_inner, *exc):
                Timer().end(name)

            def __call__(self_inner, func):
                nm = name or func.__name__

                @functools.wraps(func)
                def wrapper(*a, **k):
                    with Timer().context(nm):
                        return func(*a, **k)

                return wrapper

        return _Ctx()
    func = name_or_func

    @functools.wraps(func)
    def wrapper(*a, **k):
        with Timer().context(func.__name__):
            return func(*a, **k)

    return wrapper


@contextmanager
def inverse_timer(name: str):
    """Pause an enclosing timer ``name`` for the duration of the block (used to exclude waits)."""
    t = Timer()
    assert name in t.start_time, f"timer {name} is not running"
    t.end(name)
    try:
        yield
    finally:
        t.start(name)
