"""Heartbeats and health checking.

* ``SimpleHeartbeat``: a monotonically bumped counter + timestamp that every trainer phase touches
  (reference: miles/ray/train_actor.py:142-144).
* ``SimpleHealthChecker``: polls a probe with an interval, debounces ``failure_threshold`` consecutive
  failures before declaring the target unhealthy, and calls back once per transition
  (reference: miles/utils/ft_utils/health_checker.py:18-247).
* ``HealthMonitor``: per engine group thread that calls ``health_generate`` after ``first_wait`` every
  ``interval`` seconds with a ``timeout``; on failure the engine is marked stopped and its kill callback
  is invoked; paused while the engines are offloaded (reference: miles/utils/health_monitor.py:11-167;
  flags ``--rollout-health-check-{first-wait,interval,timeout}``).
"""
from __future__ import annotations

import threading
import time
from typing import Callable, Optional, Sequence


class SimpleHeartbeat:
    def __init__(self, clock: Callable[[], float] = time.monotonic):
        self.clock = clock
        self.count = 0
        self.last = clock()
        self.phase = "init"

    def bump(self, phase: str = "") -> None:
        self.count += 1
        self.last = self.clock()
        if phase:
            self.phase = phase

    def age(self) -> float:
        return self.clock() - self.last

    def status(self) -> dict:
        return {"count": self.count, "age": self.age(), "phase": self.phase}


class SimpleHealthChecker:
    def __init__(self, probe: Callable[[], bool], on_unhealthy: Optional[Callable[[], None]] = None,
                 on_recovered: Optional[Callable[[], None]] = None, failure_threshold: int = 3, success_threshold: int = 1):
        self.probe, self.on_unhealthy, self.on_recovered = probe, on_unhealthy, on_recovered
        self.failure_threshold, self.success_threshold = failure_threshold, success_threshold
        self.healthy = True
        self._fails = 0
        self._oks = 0

    def check_once(self) -> bool:
        try:
            ok = bool(self.probe())
        except Exception:
            ok = False
        if ok:
            self._fails = 0
            self._oks += 1
            if not self.healthy and self._oks >= self.success_threshold:
                self.healthy = True
                if self.on_recovered:
                    self.on_recovered()
        else:
            self._oks = 0
            self._fails += 1
            if self.healthy and self._fails >= self.failure_threshold:
                self.healthy = False
                if self.on_unhealthy:
                    self.on_unhealthy()
        return self.healthy


class HealthMonitor:
    """Background health checks of a list of engines (objects with ``health_generate()``)."""

    def __init__(self, engines: Sequence, kill: Callable[[int], None], first_wait: float = 0.0, interval: float = 10.0,
                 timeout: float = 30.0, sleep: Callable[[float], None] = time.sleep):
        self.engines = list(engines)
        self.kill = kill
        self.first_wait, self.interval, self.timeout = first_wait, interval, timeout
        self.sleep = sleep
        self.stopped: set = set()
        self._paused = threading.Event()
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None

    def _probe(self, i: int) -> bool:
        result: list = []

        def run():
            try:
                result.append(bool(self.engines[i].health_generate()))
            except Exception:
                result.append(False)

        t = threading.Thread(target=run, daemon=True)
        t.start()
        t.join(self.timeout)
        return bool(result and result[0])

    def check_all(self) -> list:
        failed = []
        for i in range(len(self.engines)):
            if i in self.stopped or self.engines[i] is None:
                continue
            if not self._probe(i):
                self.stopped.add(i)
                failed.append(i)
                self.kill(i)
        return failed

    def _loop(self) -> None:
        self.sleep(self.first_wait)
        while not self._stop.is_set():
            if not self._paused.is_set():
                self.check_all()
            self.sleep(self.interval)

    def start(self) -> None:
        self._thread = threading.Thread(target=self._loop, daemon=True)
        self._thread.start()

    def pause(self) -> None:
        self._paused.set()

    def resume(self) -> None:
        self._paused.clear()

    def stop(self) -> None:
        self._stop.set()

    def mark_recovered(self, i: int, engine) -> None:
        self.engines[i] = engine
        self.stopped.discard(i)
