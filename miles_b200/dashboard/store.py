"""Append-only JSONL store: one file per (stream, hour) under ``root/<stream>/<YYYYMMDD-HH>.jsonl``.

Writers append whole lines under a lock (a crash can at worst truncate the last line, which readers skip);
readers scan the partitions that overlap the requested time range.
"""
from __future__ import annotations

import json
import os
import threading
import time
from typing import Iterator, Optional


class EventStore:
    def __init__(self, root: str):
        self.root = root
        os.makedirs(root, exist_ok=True)
        self._lock = threading.Lock()

    @staticmethod
    def _partition(t: float) -> str:
        return time.strftime("%Y%m%d-%H", time.gmtime(t))

    def append(self, stream: str, record: dict, t: Optional[float] = None) -> None:
        t = time.time() if t is None else t
        d = os.path.join(self.root, stream)
        line = json.dumps({"t": t, **record}, default=str)
        with self._lock:
            os.makedirs(d, exist_ok=True)
            with open(os.path.join(d, self._partition(t) + ".jsonl"), "a") as f:
                f.write(line + "\n")

    def streams(self) -> list:
        return sorted(x for x in os.listdir(self.root) if os.path.isdir(os.path.join(self.root, x)))

    def read(self, stream: str, since: float = 0.0, until: Optional[float] = None, limit: Optional[int] = None) -> Iterator[dict]:
        d = os.path.join(self.root, stream)
        if not os.path.isdir(d):
            return
        until = time.time() + 1 if until is None else until
        lo, hi = self._partition(since), self._partition(until)
        n = 0
        for name in sorted(os.listdir(d)):
            part = name[:-6]
            if not name.endswith(".jsonl") or part < lo or part > hi:
                continue
            with open(os.path.join(d, name)) as f:
                for line in f:
                    try:
                        rec = json.loads(line)
                    except json.JSONDecodeError:
                        continue  # a torn last line
                    if since <= rec.get("t", 0) <= until:
                        yield rec
                        n += 1
                        if limit is not None and n >= limit:
                            return

    def tail(self, stream: str, n: int = 100) -> list:
        recs = list(self.read(stream, since=time.time() - 7 * 24 * 3600))
        return recs[-n:]
