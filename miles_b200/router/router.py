"""Least-inflight HTTP router with health checks and quarantine.

``/add_worker?url=...``, ``/remove_worker``, ``/list_workers`` and a catch-all proxy that forwards any
other path to the worker with the fewest in-flight requests; a background loop polls ``/health`` and
quarantines a worker after ``failure_threshold`` consecutive failures (it is re-admitted when healthy).
Reference: miles/router/router.py:34-236 (``--use-miles-router``, ``--miles-router-*`` flags).
Policies: ``least_inflight`` (default), ``round_robin``, ``consistent_hashing`` on a routing key header.
"""
import asyncio
import hashlib
import itertools
from typing import Optional


class MilesRouter:
    """Worker bookkeeping (in-flight counts, consecutive failures, quarantine) lives in the C++ ``RouterTable``
    (``csrc/native/control_plane.cpp``); this class adds the policies and the HTTP transport."""

    def __init__(self, timeout: float = 600.0, max_connections: int = 1024, failure_threshold: int = 3,
                 health_interval: float = 5.0, policy: str = "least_inflight"):
        from ..ops import _native

        self.table = _native.load().RouterTable(failure_threshold)
        self.timeout, self.max_connections = timeout, max_connections
        self.failure_threshold, self.health_interval = failure_threshold, health_interval
        self.policy = policy
        self._rr = itertools.count()
        self._client = None
        self._health_task: Optional[asyncio.Task] = None

    # ------------------------------------------------------------------ membership
    def add_worker(self, url: str) -> None:
        self.table.add(url.rstrip("/"))

    def remove_worker(self, url: str) -> None:
        self.table.remove(url.rstrip("/"))

    @property
    def workers(self) -> dict:
        """url -> requests in flight."""
        return {u: v[0] for u, v in self.table.snapshot().items()}

    @property
    def dead(self) -> set:
        return {u for u, v in self.table.snapshot().items() if v[2]}

    def live_workers(self) -> list:
        return list(self.table.urls(True))

    # ------------------------------------------------------------------ selection
    def acquire(self, routing_key: Optional[str] = None) -> str:
        """Choose a worker for one request and count it in flight; pair with :meth:`release`."""
        if self.policy == "least_inflight" or (self.policy == "consistent_hashing" and not routing_key):
            url = self.table.acquire()
            if not url:
                raise RuntimeError("no healthy worker")
            return url
        live = self.live_workers()
        if not live:
            raise RuntimeError("no healthy worker")
        if self.policy == "round_robin":
            return live[next(self._rr) % len(live)]
        ring = sorted(live, key=lambda u: hashlib.md5((u + "|" + routing_key).encode()).hexdigest())
        return ring[0]

    def release(self, url: str, ok: bool) -> None:
        self.table.release(url, ok)

    def pick(self, routing_key: Optional[str] = None) -> str:
        """Like :meth:`acquire` but without keeping the request counted (inspection, tests)."""
        url = self.acquire(routing_key)
        if self.policy == "least_inflight" or (self.policy == "consistent_hashing" and not routing_key):
            self.table.cancel(url)
        return url

    def mark_result(self, url: str, ok: bool) -> None:
        self.table.report_health(url, ok)

    # ------------------------------------------------------------------ transport
    async def _http(self):
        if self._client is None:
            import httpx

            self._client = httpx.AsyncClient(timeout=self.timeout, limits=httpx.Limits(max_connections=self.max_connections))
        return self._client

    async def forward(self, method: str, path: str, body: bytes, headers: dict):
        url = self.acquire(headers.get("x-smg-routing-key"))
        ok = False
        try:
            c = await self._http()
            r = await c.request(method, url + path, content=body, headers={"content-type": headers.get("content-type", "application/json")})
            ok = r.status_code < 500
            return r.status_code, r.content, r.headers.get("content-type", "application/json")
        finally:
            self.release(url, ok)

    async def health_loop(self) -> None:
        while True:
            c = await self._http()
            for url in list(self.table.urls(False)):
                try:
                    r = await c.get(url + "/health", timeout=5.0)
                    ok = r.status_code == 200
                except Exception:
                    ok = False
                if ok:
                    self.table.readmit(url)
                else:
                    self.mark_result(url, False)
            await asyncio.sleep(self.health_interval)


def build_router_app(router: MilesRouter):
    from fastapi import FastAPI, HTTPException, Request
    from fastapi.responses import Response

    app = FastAPI(title="miles_b200 router")

    @app.on_event("startup")
    async def _start():
        router._health_task = asyncio.create_task(router.health_loop())

    @app.post("/add_worker")
    async def add_worker(url: str):
        router.add_worker(url)
        return {"workers": list(router.workers)}

    @app.post("/remove_worker")
    async def remove_worker(url: str):
        router.remove_worker(url)
        return {"workers": list(router.workers)}

    @app.get("/list_workers")
    async def list_workers():
        return {"urls": list(router.workers), "dead": sorted(router.dead), "inflight": dict(router.workers)}

    @app.api_route("/{path:path}", methods=["GET", "POST", "PUT", "DELETE"])
    async def proxy(path: str, req: Request):
        try:
            status, content, ctype = await router.forward(req.method, "/" + path, await req.body(), dict(req.headers))
        except RuntimeError as e:
            raise HTTPException(503, str(e))
        return Response(content=content, status_code=status, media_type=ctype)

    return app


def main(argv=None) -> None:
    """``python -m miles_b200.router.router --port 3000 --worker http://127.0.0.1:30000 --worker ...``"""
    import argparse

    import uvicorn

    ap = argparse.ArgumentParser(description=main.__doc__)
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=3000)
    ap.add_argument("--worker", action="append", default=[])
    ap.add_argument("--policy", default="least_inflight", choices=["least_inflight", "round_robin", "consistent_hashing"])
    ap.add_argument("--failure-threshold", type=int, default=3)
    ap.add_argument("--health-interval", type=float, default=5.0)
    ap.add_argument("--timeout", type=float, default=600.0, help="seconds a forwarded request may take")
    ap.add_argument("--max-connections", type=int, default=1024)
    ns = ap.parse_args(argv)
    router = MilesRouter(timeout=ns.timeout, max_connections=ns.max_connections, failure_threshold=ns.failure_threshold,
                         health_interval=ns.health_interval, policy=ns.policy)
    for w in ns.worker:
        router.add_worker(w)
    uvicorn.run(build_router_app(router), host=ns.host, port=ns.port, log_level="warning")


if __name__ == "__main__":
    main()
