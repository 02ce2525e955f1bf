"""Fault-tolerance runtime of one training job (``--use-fault-tolerance``).

The reference runs trainer cells as groups of Ray actors under a controller (miles/ray/train_group_v2.py,
miles/utils/ft_utils/). A job here is SPMD, so the job's own ranks are one cell; what this module adds to the loop:

* training steps go through :class:`~miles_b200.ft.cells.TrainGroup` (retry on the survivors, discarded steps leave
  weights and optimizer state untouched) with the job's trainer wrapped as the cell's actor;
* the control server (``--control-server-port``; first rank): cell listing, suspend / resume, host-side fault injection
  (miles/utils/ft_utils/control_server/server.py);
* the mini controller (``--mini-ft-controller-enable``, ``--mini-ft-controller-poll-interval``,
  ``--mini-ft-controller-resume-delay``): suspends a cell whose heartbeat is stale, resumes it after a back-off;
* engine health monitoring for a launched fleet (``--rollout-health-check-first-wait/-interval/-timeout``);
* scripted actions of CI chaos runs (``--ci-ft-test-actions``: stop / start a cell at the end of a rollout, crash a
  rank before the gradient reduction; always a host-side exception, never a device fault).

``--ft-components`` restricts which of ``train`` / ``rollout`` get this treatment (default: both).
"""
from __future__ import annotations

import json
import threading
import time
from typing import Optional

from .cells import StepResult, TrainGroup
from .control_server import MiniFTController, build_control_app
from .fault_injector import InjectedFault, inject
from .health import SimpleHeartbeat


def parse_ci_actions(spec) -> list:
    """``--ci-ft-test-actions``: JSON array of ``{"at_rollout": N, "action": "stop_cell_at_end" | "start_cell_at_end" |
    "crash_before_allreduce", "cell_index": I, "rank": 0, "attempt": 0}`` (cell_index -1 = last cell)."""
    if not spec:
        return []
    acts = json.loads(spec) if isinstance(spec, str) else list(spec)
    for a in acts:
        assert a.get("action") in ("stop_cell_at_end", "start_cell_at_end", "crash_before_allreduce"), a
        a.setdefault("cell_index", 0)
        a.setdefault("rank", 0)
        a.setdefault("attempt", 0)
    return acts


class LoopCellActor:
    """The job's trainer behind the actor protocol a :class:`TrainCell` drives."""

    def __init__(self, runtime: "FTRuntime"):
        self.rt = runtime

    def init(self, quorum_id: int = 0) -> None:
        self.rt.quorum_id = quorum_id

    def reconfigure(self, quorum_id: int = 0, members=None) -> None:
        self.rt.quorum_id = quorum_id

    def send_ckpt(self):
        return None  # a single cell has nobody to heal from: a failed step is discarded and retried in place

    def recv_ckpt(self, ckpt) -> None:
        pass

    def inject_fault(self, kind: str) -> None:
        self.rt.pending_fault = kind

    def discard_step(self, rollout_id: int) -> None:
        actor = self.rt.loop.actor
        actor.store.zero_grads()
        if getattr(actor, "witness", None) is not None:
            actor.witness.discard()

    def train(self, rollout_id: int, data, attempt: int = 0) -> StepResult:
        rt = self.rt
        rt.heartbeat.bump("train")
        for a in rt.actions:
            if (a["action"] == "crash_before_allreduce" and a["at_rollout"] == rollout_id and a["attempt"] == attempt
                    and a["rank"] == rt.loop.ps.rank and not a.get("_done")):
                a["_done"] = True
                raise InjectedFault(f"scripted crash before the gradient reduction of rollout {rollout_id}")
        if rt.pending_fault:
            kind, rt.pending_fault = rt.pending_fault, None
            inject(kind)
        return StepResult("NORMAL", rt.loop._train_once(rollout_id, data))


class FTRuntime:
    def __init__(self, loop, args):
        self.loop, self.args = loop, args
        comps = getattr(args, "ft_components", None)
        self.components = set(comps.split(",")) if isinstance(comps, str) else set(comps or ("train", "rollout"))
        self.heartbeat = SimpleHeartbeat()
        self.quorum_id = 0
        self.pending_fault: Optional[str] = None
        self.actions = parse_ci_actions(getattr(args, "ci_ft_test_actions", None))
        self.group = TrainGroup(1, lambda i: [LoopCellActor(self)])
        self.group.init()
        self.controller: Optional[MiniFTController] = None
        self._threads: list = []
        self._stop = threading.Event()
        self.engine_monitor = None
        self.server = None
        if "train" in self.components and getattr(args, "mini_ft_controller_enable", False):
            self.controller = MiniFTController(self.group, self._cell_healthy,
                                               poll_interval=float(getattr(args, "mini_ft_controller_poll_interval", 10.0)),
                                               resume_delay=float(getattr(args, "mini_ft_controller_resume_delay", 10.0)))
            t = threading.Thread(target=self._controller_loop, name="mini-ft-controller", daemon=True)
            t.start()
            self._threads.append(t)
        port = int(getattr(args, "control_server_port", 0) or 0)
        if port > 0 and loop.ps.rank == 0:
            self._start_control_server(port)
        if "rollout" in self.components and getattr(loop, "fleet", None) is not None:
            self.engine_monitor = loop.fleet.monitor(interval=float(getattr(args, "rollout_health_check_interval", 30.0)),
                                                     timeout=float(getattr(args, "rollout_health_check_timeout", 30.0)),
                                                     recover=True, on_recovered=self._engine_recovered)
            self.engine_monitor.first_wait = float(getattr(args, "rollout_health_check_first_wait", 0) or 0)
            self.engine_monitor.start()

    # ------------------------------------------------------------------ training through the cell group
    def train(self, rollout_id: int, data) -> dict:
        """One training step with retries; a suspended cell trains nothing (its samples are dropped, as for a cell that
        is down in the reference) and reports so."""
        if self.group.cells[0].suspended:
            return {"train/skipped_suspended": 1.0}
        res = self.group.train_step(rollout_id, lambda rank, n: data)
        return res[0][0].payload

    def after_rollout(self, rollout_id: int) -> None:
        self.heartbeat.bump("rollout_end")
        n = len(self.group.cells)
        for a in self.actions:
            if a["at_rollout"] != rollout_id or a.get("_done"):
                continue
            cell = a["cell_index"] % n
            if a["action"] == "stop_cell_at_end":
                self.group.suspend(cell)
                a["_done"] = True
            elif a["action"] == "start_cell_at_end":
                self.group.resume(cell)
                self.group.refresh_cells()
                a["_done"] = True

    # ------------------------------------------------------------------ helpers
    def _cell_healthy(self, index: int) -> bool:
        limit = 3.0 * float(getattr(self.args, "mini_ft_controller_poll_interval", 10.0)) + 600.0
        return self.heartbeat.age() < limit

    def _controller_loop(self) -> None:
        while not self._stop.wait(self.controller.poll_interval):
            try:
                self.controller.poll_once()
                self.group.refresh_cells()
            except Exception:  # noqa: BLE001 - the controller must outlive one bad poll
                pass

    def _start_control_server(self, port: int) -> None:
        import uvicorn

        cfg = uvicorn.Config(build_control_app(self.group), host="127.0.0.1", port=port, log_level="warning")
        self.server = uvicorn.Server(cfg)
        t = threading.Thread(target=self.server.run, name="ft-control-server", daemon=True)
        t.start()
        self._threads.append(t)
        deadline = time.time() + 10
        while not self.server.started and time.time() < deadline:
            time.sleep(0.05)

    def _engine_recovered(self, index: int, url: str) -> None:
        upd = getattr(self.loop, "weight_updater", None)
        if upd is not None and hasattr(upd, "replace_engine"):
            upd.replace_engine(index, url)

    def stop(self) -> None:
        self._stop.set()
        if self.engine_monitor is not None:
            self.engine_monitor.stop()
        if self.server is not None:
            self.server.should_exit = True
