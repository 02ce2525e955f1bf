"""Evaluation that does not block the training loop.

``EvalDispatcher.dispatch(rollout_id)`` starts an evaluation in the background (at most one at a time: a new
request while one is running is skipped unless ``force``), optionally on a *snapshot*: the weights are first
exported to a directory (``export_fn``) so that training can move on while the evaluation reads the files, and the
directory is deleted when the evaluation settles. ``drain()`` waits for what is in flight; finished results are
handed to ``on_result(rollout_id, metrics)`` in dispatch order.

``CheckpointEvalFn`` is the base class of user evaluators that score a checkpoint directory with their own harness
(a dedicated engine fleet, an external service): subclass it, implement ``evaluate_checkpoint`` and point
``--eval-function-path`` at the class.

Reference counterpart: miles/ray/rollout/eval_dispatch.py:12-95 and miles/rollout/checkpoint_eval.py:35-85.
"""
from __future__ import annotations

import abc
import asyncio
import shutil
import time
from typing import Awaitable, Callable, Optional


class EvalSkip(Exception):
    """Raised by an evaluator to say "nothing to report for this checkpoint" (not an error)."""

    def __init__(self, reason: str):
        super().__init__(reason)
        self.reason = reason


class CheckpointEvalFn(abc.ABC):
    def __init__(self, args):
        self.args = args

    @abc.abstractmethod
    async def evaluate_checkpoint(self, checkpoint_dir: str, rollout_id: int) -> dict: ...

    async def __call__(self, checkpoint_dir: str, rollout_id: int) -> dict:
        try:
            return await self.evaluate_checkpoint(checkpoint_dir, rollout_id)
        except EvalSkip as e:
            return {"eval/skipped": 1.0, "eval/skip_reason": e.reason}

    def dispose(self) -> None:  # optional hook
        return None


def is_checkpoint_eval_fn(obj) -> bool:
    return isinstance(obj, type) and issubclass(obj, CheckpointEvalFn)


class EvalDispatcher:
    """``max_in_flight`` evaluations may run at once (``--eval-max-in-flight``); a request beyond that waits for the
    oldest one (``overflow_policy="backpressure"``) or is dropped and recorded in ``skipped`` (``"skip"``,
    ``--eval-overflow-policy``). ``keep_snapshots`` newest export directories stay on disk after their evaluation
    (``--eval-keep-snapshots``; 0 deletes each one as soon as it is scored)."""

    def __init__(self, eval_fn: Callable[..., Awaitable[dict]], export_fn: Optional[Callable[[int, str], Awaitable[None]]] = None,
                 on_result: Optional[Callable[[int, dict], None]] = None, keep_exports: bool = False, max_in_flight: int = 1,
                 overflow_policy: str = "backpressure", keep_snapshots: int = 0):
        assert overflow_policy in ("backpressure", "skip")
        self.eval_fn, self.export_fn, self.on_result = eval_fn, export_fn, on_result
        self.keep_exports = keep_exports
        self.max_in_flight, self.overflow_policy, self.keep_snapshots = max(1, int(max_in_flight)), overflow_policy, int(keep_snapshots)
        self._tasks: list = []
        self._kept: list = []
        self.results: list = []
        self.skipped: list = []

    def _prune(self) -> None:
        self._tasks = [t for t in self._tasks if not t.done()]

    @property
    def busy(self) -> bool:
        self._prune()
        return len(self._tasks) >= self.max_in_flight

    async def dispatch(self, rollout_id: int, export_dir: Optional[str] = None, force: bool = False) -> bool:
        """Returns True if an evaluation was started."""
        if self.busy:
            if not force and self.overflow_policy == "skip":
                self.skipped.append(rollout_id)
                return False
            await self._tasks[0]  # backpressure: the oldest evaluation has to settle first
            self._prune()
        exported = None
        t_export = 0.0
        if self.export_fn is not None and export_dir is not None:
            t0 = time.perf_counter()
            await self.export_fn(rollout_id, export_dir)  # the only part the training loop waits for
            t_export = time.perf_counter() - t0
            exported = export_dir
        self._tasks.append(asyncio.ensure_future(self._settle(rollout_id, exported, t_export)))
        return True

    async def _settle(self, rollout_id: int, exported: Optional[str], t_export: float) -> None:
        t0 = time.perf_counter()
        try:
            metrics = dict(await (self.eval_fn(exported, rollout_id) if exported is not None else self.eval_fn(rollout_id)))
        except EvalSkip as e:
            metrics = {"eval/skipped": 1.0, "eval/skip_reason": e.reason}
        finally:
            if exported is not None and not self.keep_exports:
                self._kept.append(exported)
                while len(self._kept) > self.keep_snapshots:
                    shutil.rmtree(self._kept.pop(0), ignore_errors=True)
        metrics["perf/eval_time"] = time.perf_counter() - t0
        metrics["perf/eval_export_time"] = t_export
        self.results.append((rollout_id, metrics))
        if self.on_result is not None:
            self.on_result(rollout_id, metrics)

    async def drain(self) -> None:
        for t in list(self._tasks):
            await t
        self._tasks = []
