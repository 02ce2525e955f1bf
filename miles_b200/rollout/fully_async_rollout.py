"""Fully-asynchronous rollout: a persistent producer keeps groups in flight across ``generate()`` calls.

Behaviour of the reference's miles/rollout/fully_async_rollout.py:51-203 and
fully_async_data_buffer.py:58-192: the producer task keeps at most ``--async-max-concurrent-samples``
samples in flight and puts finished groups into a bounded buffer (capacity =
``--async-data-buffer-capacity-factor`` x rollout batch); abort / dynamic filters run on ``put``; the
**staleness filter** runs on ``get`` (a group whose oldest weight version lags the current one by more than
``--max-weight-staleness`` is retried or dropped, ``--async-unused-samples-handler``); evaluation pauses
the producer.
"""
from __future__ import annotations

import asyncio
import time
from collections import deque
from typing import Optional

from ..utils.misc import load_function
from ..utils.types import Sample
from .base_types import RolloutFnConstructorInput, RolloutFnTrainOutput
from .generate_hub.common import GenerateState
from .inference_rollout import generate_and_rm_group


def group_oldest_version(group: list) -> Optional[int]:
    vs = [s.oldest_weight_version() for s in group]
    vs = [v for v in vs if v is not None]
    return min(vs) if vs else None


class DefaultDataBuffer:
    """Bounded FIFO of finished groups with put-side filters and a get-side staleness filter."""

    def __init__(self, args, data_source=None, dynamic_filter=None):
        self.args = args
        self.capacity = max(1, int(getattr(args, "async_data_buffer_capacity_factor", 2) * args.rollout_batch_size))
        self.max_staleness = getattr(args, "max_weight_staleness", None)
        self.unused_handler = getattr(args, "async_unused_samples_handler", "retry")
        self.data_source = data_source
        self.dynamic_filter = dynamic_filter
        self.groups: deque = deque()
        self.stats = {"put": 0, "dropped_abort": 0, "dropped_filter": 0, "dropped_stale": 0, "retried_stale": 0}
        self._not_full = asyncio.Event()
        self._not_full.set()

    def __len__(self) -> int:
        return len(self.groups)

    def full(self) -> bool:
        return len(self.groups) >= self.capacity

    async def wait_for_space(self) -> None:
        while self.full():
            self._not_full.clear()
            await self._not_full.wait()

    def put(self, group: list) -> bool:
        if any(s.status == Sample.Status.ABORTED for s in group):
            self.stats["dropped_abort"] += 1
            return False
        if self.dynamic_filter is not None:
            v = self.dynamic_filter(self.args, group)
            if not (v.keep if hasattr(v, "keep") else bool(v)):
                self.stats["dropped_filter"] += 1
                return False
        self.groups.append(group)
        self.stats["put"] += 1
        return True

    def _is_stale(self, group: list, current_version: int) -> bool:
        if self.max_staleness is None:
            return False
        oldest = group_oldest_version(group)
        return oldest is not None and current_version - oldest > self.max_staleness

    def _recycle(self, group: list) -> None:
        if self.unused_handler == "retry" and self.data_source is not None:
            fresh = []
            for s in group:
                t = s.clone()
                t.tokens, t.response, t.response_length = list(t.tokens[:t.prompt_length]), "", 0
                t.reward, t.loss_mask, t.rollout_log_probs, t.rollout_routed_experts = None, None, None, None
                t.weight_versions, t.status = [], Sample.Status.PENDING
                fresh.append(t)
            self.data_source.add_samples([fresh])
            self.stats["retried_stale"] += 1
        else:
            self.stats["dropped_stale"] += 1

    def get(self, n: int, current_version: int) -> list:
        """Up to ``n`` fresh-enough groups in FIFO order; stale ones are recycled or dropped."""
        out = []
        while self.groups and len(out) < n:
            g = self.groups.popleft()
            if self._is_stale(g, current_version):
                self._recycle(g)
                continue
            out.append(g)
        self._not_full.set()
        return out


class FullyAsyncRolloutFn:
    def __init__(self, inp: RolloutFnConstructorInput):
        self.args = inp.args
        self.data_source = inp.data_source
        self.state = GenerateState(inp.args, inp.engine_client, getattr(inp.engine_client, "tokenizer", None))
        p = getattr(self.args, "dynamic_sampling_filter_path", None)
        flt = load_function(p) if p else None
        bp = getattr(self.args, "custom_async_data_buffer_path", None)
        buf_cls = load_function(bp) if bp else DefaultDataBuffer
        self.buffer = buf_cls(self.args, self.data_source, flt)
        n = self.args.n_samples_per_prompt
        max_samples = getattr(self.args, "async_max_concurrent_samples", None) or 2 * self.args.rollout_batch_size * n
        self.max_groups_in_flight = max(1, max_samples // n)
        self.in_flight: set = set()
        self.producer: Optional[asyncio.Task] = None
        self.paused = False
        self._loop: Optional[asyncio.AbstractEventLoop] = None

    # The producer lives on a private event loop that ``__call__`` drives, so that it survives between calls.
    def _ensure_loop(self) -> asyncio.AbstractEventLoop:
        if self._loop is None or self._loop.is_closed():
            self._loop = asyncio.new_event_loop()
        return self._loop

    async def _produce(self) -> None:
        while True:
            if self.paused:
                await asyncio.sleep(0.001)
                continue
            await self.buffer.wait_for_space()
            while len(self.in_flight) < self.max_groups_in_flight and not self.paused:
                for group in self.data_source.get_samples(1):
                    t = asyncio.ensure_future(generate_and_rm_group(self.state, group, self.state.sampling_params))
                    self.in_flight.add(t)
            if not self.in_flight:
                await asyncio.sleep(0.001)
                continue
            done, _ = await asyncio.wait(self.in_flight, return_when=asyncio.FIRST_COMPLETED, timeout=0.05)
            for t in done:
                self.in_flight.discard(t)
                try:
                    self.buffer.put(t.result())
                except Exception:
                    continue

    async def _collect(self, rollout_id: int) -> RolloutFnTrainOutput:
        if self.producer is None or self.producer.done():
            self.producer = asyncio.ensure_future(self._produce())
        target = self.args.rollout_batch_size
        data: list = []
        t0 = time.perf_counter()
        # multi-adapter service: train on what is ready once ``rollout_coalesce_wait_s`` have passed since the first group
        # arrived; fail if not a single group arrives within ``rollout_empty_wait_s`` (0 = wait for the full batch forever)
        coalesce = float(getattr(self.args, "rollout_coalesce_wait_s", 0.0) or 0.0)
        empty_wait = float(getattr(self.args, "rollout_empty_wait_s", 0.0) or 0.0)
        t_first = None
        while len(data) < target:
            data += self.buffer.get(target - len(data), self.state.client.weight_version())
            if data and t_first is None:
                t_first = time.perf_counter()
            if len(data) < target:
                now = time.perf_counter()
                if coalesce and t_first is not None and now - t_first >= coalesce:
                    break
                if empty_wait and not data and now - t0 >= empty_wait:
                    raise TimeoutError(f"no finished rollout group within {empty_wait:.0f} s")
                await asyncio.sleep(0.001)
        data.sort(key=lambda g: g[0].index or 0)
        m = {f"rollout/async_buffer/{k}": v for k, v in self.buffer.stats.items()}
        m["rollout/async_buffer/size"] = len(self.buffer)
        m["perf/rollout_wait_time"] = time.perf_counter() - t0
        return RolloutFnTrainOutput(samples=data, metrics=m)

    def __call__(self, inp):
        loop = self._ensure_loop()
        if inp.evaluation:
            from .eval import eval_rollout

            self.paused = True
            try:
                return loop.run_until_complete(eval_rollout(self.args, self.state, inp.rollout_id))
            finally:
                self.paused = False
        return loop.run_until_complete(self._collect(inp.rollout_id))

    def pump(self, seconds: float) -> None:
        """Let the producer make progress for a while (called between trainer phases in the async driver)."""
        loop = self._ensure_loop()
        if self.producer is None or self.producer.done():
            self.producer = loop.create_task(self._produce())
        loop.run_until_complete(asyncio.sleep(seconds))

    def shutdown(self) -> None:
        if self._loop is not None and not self._loop.is_closed():
            for t in list(self.in_flight) + ([self.producer] if self.producer else []):
                t.cancel()
            self._loop.run_until_complete(asyncio.sleep(0))
            self._loop.close()
