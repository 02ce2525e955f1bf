"""Pacing of prompt-group submission to the engine (``--rollout-submission-granularity group|sample``).

``group``: a slot frees when a whole group (all samples of one prompt) has returned, so at most ``budget`` groups are
in flight. ``sample``: every finished sample frees its own slot and a new group is admitted as soon as a group's
worth of slots is free, which keeps the engine's batch full while stragglers of old groups are still decoding.

Reference: miles/rollout/submission_scheduler.py:16-71.
"""
from __future__ import annotations

import asyncio
from typing import Iterable


class SubmissionPacer:
    def __init__(self, granularity: str, group_size: int):
        assert granularity in ("group", "sample"), f"unknown submission granularity: {granularity}"
        self.by_sample = granularity == "sample"
        self.group_size = max(1, group_size)
        self.samples_in_flight = 0
        self._progress = asyncio.Event()

    # called by the generate wrapper of every sample (sample mode only)
    def sample_finished(self) -> None:
        if self.by_sample:
            self.samples_in_flight = max(0, self.samples_in_flight - 1)
            self._progress.set()

    def submitted(self, groups: Iterable) -> None:
        if self.by_sample:
            self.samples_in_flight += sum(len(g) for g in groups)

    def may_submit(self, pending_groups: int, group_budget: int) -> bool:
        if not self.by_sample:
            return pending_groups < group_budget
        if pending_groups == 0:
            self.samples_in_flight = 0  # nothing can be running: drop a stale count rather than stall
        if self.samples_in_flight + self.group_size <= group_budget * self.group_size:
            return True
        self._progress.clear()  # from here on only a later completion wakes the waiter
        return False

    async def wait(self, pending: set) -> tuple:
        """Block until a group task finishes or (sample mode) a sample frees a slot; returns (done, still pending)."""
        if not self.by_sample:
            return await asyncio.wait(pending, return_when=asyncio.FIRST_COMPLETED)
        waker = asyncio.ensure_future(self._progress.wait())
        try:
            done, rest = await asyncio.wait(set(pending) | {waker}, return_when=asyncio.FIRST_COMPLETED)
        finally:
            waker.cancel()
        return done - {waker}, rest - {waker}


def make_pacer(args, default: str = "group") -> SubmissionPacer:
    return SubmissionPacer(getattr(args, "rollout_submission_granularity", None) or default, args.n_samples_per_prompt)
