"""Trainer cells: one independent data-parallel replica per cell, with a retrying group on top.

State machine (reference: miles/ray/train/cell_state.py:11-37, cell.py:29-303, group.py:42-491)::

    Pending -> AllocatedUninitialized -> AllocatedAlive -> (Errored | Stopped) -> Pending ...

``TrainCell.execute`` fans a call out to the cell's actors; any exception marks the cell errored and
kills its actors.  ``TrainGroup.train_step`` retries a step (at most ``max_retries`` times) on the
surviving cells and accepts it only if every alive cell returned normally; ``refresh_cells`` bumps the
quorum id, allocates pending cells, lets the survivors reconfigure their cross-cell process groups
under the new quorum and streams an in-memory checkpoint from one survivor to each healed cell.
Actors are plain Python objects behind a factory, so the logic is testable with dummy actors on CPU.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass
from typing import Any, Callable, Optional


class CellState(enum.Enum):
    PENDING = "pending"
    ALLOCATED_UNINITIALIZED = "allocated_uninitialized"
    ALLOCATED_ALIVE = "allocated_alive"
    ERRORED = "errored"
    STOPPED = "stopped"


@dataclass
class StepResult:
    status: str = "NORMAL"      # NORMAL | DISCARDED
    payload: Any = None


class TrainCell:
    def __init__(self, index: int, actor_factory: Callable[[int], list]):
        self.index = index
        self.actor_factory = actor_factory
        self.actors: list = []
        self.state = CellState.PENDING
        self.last_error: Optional[BaseException] = None
        self.suspended = False

    @property
    def alive(self) -> bool:
        return self.state == CellState.ALLOCATED_ALIVE

    def allocate(self) -> None:
        assert self.state == CellState.PENDING, f"cell {self.index} is {self.state}"
        self.actors = self.actor_factory(self.index)
        self.state = CellState.ALLOCATED_UNINITIALIZED

    def mark_alive(self) -> None:
        assert self.state == CellState.ALLOCATED_UNINITIALIZED
        self.state = CellState.ALLOCATED_ALIVE

    def _kill(self) -> None:
        for a in self.actors:
            kill = getattr(a, "kill", None)
            if kill:
                try:
                    kill()
                except Exception:
                    pass
        self.actors = []

    def stop(self) -> None:
        self._kill()
        self.state = CellState.STOPPED

    def mark_pending(self) -> None:
        assert self.state in (CellState.ERRORED, CellState.STOPPED)
        self.state = CellState.PENDING
        self.last_error = None

    def execute(self, method: str, *args, **kwargs) -> list:
        assert self.state in (CellState.ALLOCATED_ALIVE, CellState.ALLOCATED_UNINITIALIZED), f"cell {self.index} is {self.state}"
        try:
            return [getattr(a, method)(*args, **kwargs) for a in self.actors]
        except BaseException as e:  # noqa: BLE001 - any actor failure takes the cell down
            self.last_error = e
            self._kill()
            self.state = CellState.ERRORED
            raise


class TrainGroup:
    def __init__(self, num_cells: int, actor_factory: Callable[[int], list], max_retries: int = 30,
                 heartbeat_timeout: float = 60.0):
        self.cells = [TrainCell(i, actor_factory) for i in range(num_cells)]
        self.max_retries = max_retries
        self.quorum_id = 0
        self.events: list = []
        # membership as the participants would see it through the C++ quorum store (csrc/native/control_plane.cpp):
        # members that stop heartbeating drop out after `heartbeat_timeout` even if nobody reports them
        from ..ops import _native

        self.store = _native.load().QuorumStore(timeout_s=heartbeat_timeout)

    def alive_cells(self) -> list:
        return [c for c in self.cells if c.alive]

    def init(self) -> None:
        self.refresh_cells(initial=True)

    def refresh_cells(self, initial: bool = False) -> None:
        """Heal: bump the quorum, (re)allocate pending cells, reconfigure survivors, transfer a checkpoint."""
        for c in self.cells:
            if c.state in (CellState.ERRORED, CellState.STOPPED) and not c.suspended:
                c.mark_pending()
        pending = [c for c in self.cells if c.state == CellState.PENDING and not c.suspended]
        survivors = self.alive_cells()
        if not pending and not initial:
            return
        self.quorum_id += 1
        for c in pending:
            c.allocate()
        for c in pending:
            try:
                c.execute("init", quorum_id=self.quorum_id)
            except BaseException:
                continue
        members = [c.index for c in survivors] + [c.index for c in pending if c.state == CellState.ALLOCATED_UNINITIALIZED]
        for c in self.cells:
            if c.index in members:
                self.store.heartbeat(f"cell-{c.index}")
            else:
                self.store.evict(f"cell-{c.index}")
        for c in survivors:
            try:
                c.execute("reconfigure", quorum_id=self.quorum_id, members=members)
            except BaseException:
                pass
        donor = next((c for c in survivors if c.alive), None)
        for c in pending:
            if c.state != CellState.ALLOCATED_UNINITIALIZED:
                continue
            try:
                if donor is not None:
                    ckpt = donor.execute("send_ckpt")[0]
                    c.execute("recv_ckpt", ckpt)
                c.execute("reconfigure", quorum_id=self.quorum_id, members=members)
                c.mark_alive()
                self.events.append(("healed", c.index, self.quorum_id))
            except BaseException:
                continue

    def train_step(self, rollout_id: int, data_per_cell: Callable[[int, int], Any]) -> list:
        """Run one step on all alive cells, retrying on the survivors when a cell fails mid-step."""
        for attempt in range(self.max_retries):
            alive = self.alive_cells()
            if not alive:
                self.refresh_cells()
                alive = self.alive_cells()
                if not alive:
                    raise RuntimeError("no alive trainer cell")
            results, failed = {}, False
            for rank, c in enumerate(alive):
                try:
                    results[c.index] = c.execute("train", rollout_id, data_per_cell(rank, len(alive)), attempt=attempt)
                except BaseException as e:  # noqa: BLE001
                    self.events.append(("cell_error", c.index, repr(e)))
                    failed = True
            ok = not failed and all(getattr(r, "status", "NORMAL") == "NORMAL" for rs in results.values() for r in rs)
            if ok:
                self.events.append(("step_ok", rollout_id, attempt))
                return [results[c.index] for c in alive]
            for c in self.alive_cells():
                try:
                    c.execute("discard_step", rollout_id)
                except BaseException:
                    pass
            self.refresh_cells()
        raise RuntimeError(f"train step {rollout_id} failed {self.max_retries} times")

    def suspend(self, index: int) -> None:
        c = self.cells[index]
        c.suspended = True
        if c.state in (CellState.ALLOCATED_ALIVE, CellState.ALLOCATED_UNINITIALIZED):
            c.stop()

    def resume(self, index: int) -> None:
        self.cells[index].suspended = False

    def describe(self) -> list:
        return [{"name": f"cell-{c.index}", "state": c.state.value, "suspended": c.suspended,
                 "error": repr(c.last_error) if c.last_error else None} for c in self.cells]
