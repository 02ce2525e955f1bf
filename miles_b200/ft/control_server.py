"""Control plane for trainer cells: a small K8s-style HTTP API plus an in-process mini controller.

``GET /api/v1/cells``, ``GET /api/v1/cells/{name}``, ``PATCH /api/v1/cells/{name}`` with
``{"spec": {"suspend": true|false}}`` and ``POST /api/v1/cells/{name}/inject-fault`` (host-side faults
only: ``exception``, ``exit``; the fault is delivered to the cell's actors through their ``inject_fault``
method).  ``MiniFTController`` polls cell health, suspends unhealthy cells and resumes them after a
back-off.  Reference: miles/utils/ft_utils/control_server/server.py:1-156, mini_ft_controller.py:1-221;
flags ``--control-server-port``, ``--mini-ft-controller-*``.
"""
import time
from typing import Callable

from .cells import CellState, TrainGroup


def build_control_app(group: TrainGroup):
    from fastapi import FastAPI, HTTPException, Request

    app = FastAPI(title="miles_b200 control")

    def _find(name: str):
        for i, d in enumerate(group.describe()):
            if d["name"] == name:
                return i, d
        raise HTTPException(404, f"no cell {name}")

    def _resource(d: dict) -> dict:
        ready = d["state"] == CellState.ALLOCATED_ALIVE.value
        return {"kind": "Cell", "metadata": {"name": d["name"]}, "spec": {"suspend": d["suspended"]},
                "status": {"phase": d["state"], "conditions": [{"type": "Ready", "status": "True" if ready else "False",
                                                                  "reason": d["error"] or d["state"]}]}}

    @app.get("/api/v1/cells")
    async def list_cells():
        return {"kind": "CellList", "items": [_resource(d) for d in group.describe()]}

    @app.get("/api/v1/cells/{name}")
    async def get_cell(name: str):
        return _resource(_find(name)[1])

    @app.patch("/api/v1/cells/{name}")
    async def patch_cell(name: str, req: Request):
        i, _ = _find(name)
        body = await req.json()
        suspend = (body.get("spec") or {}).get("suspend")
        if suspend is True:
            group.suspend(i)
        elif suspend is False:
            group.resume(i)
        return _resource(group.describe()[i])

    @app.post("/api/v1/cells/{name}/inject-fault")
    async def inject_fault(name: str, req: Request):
        i, _ = _find(name)
        body = await req.json()
        kind = body.get("type", "exception")
        if kind not in ("exception", "exit"):
            raise HTTPException(400, "only host-side faults (exception, exit) can be injected")
        delivered = 0
        for a in group.cells[i].actors:
            fn = getattr(a, "inject_fault", None)
            if fn:
                fn(kind)
                delivered += 1
        return {"delivered": delivered}

    return app


class MiniFTController:
    def __init__(self, group: TrainGroup, is_healthy: Callable[[int], bool], poll_interval: float = 5.0, resume_delay: float = 30.0,
                 clock: Callable[[], float] = time.monotonic):
        self.group, self.is_healthy = group, is_healthy
        self.poll_interval, self.resume_delay, self.clock = poll_interval, resume_delay, clock
        self.suspended_at: dict = {}
        self.backoff: dict = {}

    def poll_once(self) -> None:
        now = self.clock()
        for c in self.group.cells:
            if c.alive and not self.is_healthy(c.index):
                self.group.suspend(c.index)
                self.suspended_at[c.index] = now
                self.backoff[c.index] = min(self.backoff.get(c.index, self.resume_delay) * 2, 16 * self.resume_delay) \
                    if c.index in self.backoff else self.resume_delay
            elif c.suspended and c.index in self.suspended_at and now - self.suspended_at[c.index] >= self.backoff[c.index]:
                self.group.resume(c.index)
                del self.suspended_at[c.index]
