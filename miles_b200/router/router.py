"""Least-inflight HTTP router with health checks and quarantine.

``/add_worker?url=...``, ``/remove_worker``, ``/list_workers`` and a catch-all proxy that forwards any
other path to the worker with the fewest in-flight requests; a background loop polls ``/health`` and
quarantines a worker after ``failure_threshold`` consecutive failures (it is re-admitted when healthy).
Reference: miles/router/router.py:34-236 (``--use-miles-router``, ``--miles-router-*`` flags).
Policies: ``least_inflight`` (default), ``round_robin``, ``consistent_hashing`` on a routing key header.
"""
from __future__ import annotations

import asyncio
import hashlib
import itertools
from typing import Optional


class MilesRouter:
    def __init__(self, timeout: float = 600.0, max_connections: int = 1024, failure_threshold: int = 3,
                 health_interval: float = 5.0, policy: str = "least_inflight"):
        self.workers: dict = {}          # url -> in-flight count
        self.failures: dict = {}
        self.dead: set = set()
        self.timeout, self.max_connections = timeout, max_connections
        self.failure_threshold, self.health_interval = failure_threshold, health_interval
        self.policy = policy
        self._rr = itertools.count()
        self._client = None
        self._health_task: Optional[asyncio.Task] = None

    # ------------------------------------------------------------------ membership
    def add_worker(self, url: str) -> None:
        url = url.rstrip("/")
        self.workers.setdefault(url, 0)
        self.failures[url] = 0
        self.dead.discard(url)

    def remove_worker(self, url: str) -> None:
        url = url.rstrip("/")
        self.workers.pop(url, None)
        self.failures.pop(url, None)
        self.dead.discard(url)

    def live_workers(self) -> list:
        return [u for u in self.workers if u not in self.dead]

    # ------------------------------------------------------------------ selection
    def pick(self, routing_key: Optional[str] = None) -> str:
        live = self.live_workers()
        if not live:
            raise RuntimeError("no healthy worker")
        if self.policy == "round_robin":
            return live[next(self._rr) % len(live)]
        if self.policy == "consistent_hashing" and routing_key:
            ring = sorted(live, key=lambda u: hashlib.md5((u + "|" + routing_key).encode()).hexdigest())
            return ring[0]
        return min(live, key=lambda u: self.workers[u])

    def mark_result(self, url: str, ok: bool) -> None:
        if ok:
            self.failures[url] = 0
            return
        self.failures[url] = self.failures.get(url, 0) + 1
        if self.failures[url] >= self.failure_threshold:
            self.dead.add(url)

    # ------------------------------------------------------------------ transport
    async def _http(self):
        if self._client is None:
            import httpx

            self._client = httpx.AsyncClient(timeout=self.timeout, limits=httpx.Limits(max_connections=self.max_connections))
        return self._client

    async def forward(self, method: str, path: str, body: bytes, headers: dict):
        url = self.pick(headers.get("x-smg-routing-key"))
        self.workers[url] += 1
        try:
            c = await self._http()
            r = await c.request(method, url + path, content=body, headers={"content-type": headers.get("content-type", "application/json")})
            self.mark_result(url, r.status_code < 500)
            return r.status_code, r.content, r.headers.get("content-type", "application/json")
        except Exception:
            self.mark_result(url, False)
            raise
        finally:
            if url in self.workers:
                self.workers[url] -= 1

    async def health_loop(self) -> None:
        while True:
            c = await self._http()
            for url in list(self.workers):
                try:
                    r = await c.get(url + "/health", timeout=5.0)
                    ok = r.status_code == 200
                except Exception:
                    ok = False
                if ok and url in self.dead:
                    self.dead.discard(url)
                    self.failures[url] = 0
                elif not ok:
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
