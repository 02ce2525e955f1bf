"""Host-side fault injection for tests and chaos runs: an exception, a process exit, a SIGKILL of the own
process or a Python-level deadlock of a helper thread.  No GPU fault is ever produced
(reference: miles/utils/test_utils/fault_injector.py:15-41; scripted actions ft_test_actions.py:15-100)."""
from __future__ import annotations

import os
import signal
import threading
from dataclasses import dataclass


class InjectedFault(RuntimeError):
    pass


def inject(kind: str) -> None:
    if kind == "exception":
        raise InjectedFault("injected fault")
    if kind == "exit":
        os._exit(17)
    if kind == "sigkill":
        os.kill(os.getpid(), signal.SIGKILL)
    if kind == "deadlock":
        lock = threading.Lock()
        lock.acquire()
        threading.Thread(target=lock.acquire, daemon=True).start()
        return
    raise ValueError(f"unknown fault {kind!r}")


@dataclass
class ScriptedAction:
    """``stop_cell_at_end:<cell>:<rollout>``, ``start_cell_at_end:<cell>:<rollout>``, ``crash_before_allreduce:<cell>:<rollout>``."""
    kind: str
    cell: int
    rollout_id: int

    @classmethod
    def parse(cls, text: str) -> "ScriptedAction":
        kind, cell, rid = text.split(":")
        assert kind in ("stop_cell_at_end", "start_cell_at_end", "crash_before_allreduce"), kind
        return cls(kind, int(cell), int(rid))


def parse_actions(spec) -> list:
    if not spec:
        return []
    items = spec if isinstance(spec, (list, tuple)) else str(spec).split(",")
    return [ScriptedAction.parse(s.strip()) for s in items if s.strip()]
