"""Bring up the engine fleet a ``Deployment`` describes: one `miles_b200.engine.server` process per engine placement
(pinned to its GPUs through ``CUDA_VISIBLE_DEVICES``), wait until every engine answers ``/health``, hand back their
URLs per model. ``restart`` replaces one engine (what the health monitor calls after it killed an unresponsive one).

Reference counterpart: the server-group bring-up and recovery of miles/ray/rollout/rollout_server.py:17-301 and
miles/ray/rollout/server_group.py:24-274 (there as Ray actors around SGLang server processes).
"""
from __future__ import annotations

import os
import subprocess
import sys
import time
import urllib.request
from dataclasses import dataclass
from typing import Optional

from .deployment import Deployment, EnginePlacement


@dataclass
class EngineProcess:
    placement: EnginePlacement
    port: int
    proc: subprocess.Popen

    @property
    def url(self) -> str:
        return f"http://127.0.0.1:{self.port}"

    def health_generate(self, timeout: float = 30.0) -> bool:
        """One real token through the engine (what the health monitor probes)."""
        import json

        if not self.alive():
            return False
        with urllib.request.urlopen(self.url + "/health_generate", timeout=timeout) as r:
            return json.loads(r.read().decode()).get("status") in ("ok", "paused")

    def alive(self) -> bool:
        return self.proc.poll() is None


class Fleet:
    def __init__(self, deployment: Deployment, model_preset: Optional[str] = None, base_port: int = 30000,
                 device: Optional[str] = None, extra_args: Optional[list] = None, env: Optional[dict] = None, first_gpu: int = 0,
                 ports: Optional[list] = None):
        self.ports = list(ports) if ports else None  # explicit port per engine (default: base_port, base_port + 1, ...)
        self.first_gpu = first_gpu  # GPUs below this index belong to the trainer
        self.deployment, self.model_preset, self.base_port = deployment, model_preset, base_port
        self.device, self.extra_args, self.env = device, list(extra_args or []), dict(env or {})
        self.engines: list = []

    def _command(self, pl: EnginePlacement, port: int) -> list:
        cmd = [sys.executable, "-m", "miles_b200.engine.server", "--port", str(port)]
        if pl.model_path and os.path.exists(os.path.join(pl.model_path, "config.json")):
            cmd += ["--hf-checkpoint", pl.model_path]
        else:
            cmd += ["--model-preset", self.model_preset or pl.model_path or ""]
        if self.device:
            cmd += ["--device", self.device]
        for k, v in pl.overrides.items():  # ServerArgs-style overrides that the server understands
            flag = "--" + k.replace("_", "-")
            if flag in ("--max-running-requests", "--page-size", "--context-length", "--mem-fraction-static", "--quantization"):
                cmd += [flag, str(v)]
        return cmd + self.extra_args

    def _spawn(self, pl: EnginePlacement, port: int) -> EngineProcess:
        env = dict(os.environ, **self.env)
        if not (self.device or "").startswith("cpu"):
            env["CUDA_VISIBLE_DEVICES"] = ",".join(str(g) for g in pl.gpu_ids)
        return EngineProcess(pl, port, subprocess.Popen(self._command(pl, port), env=env))

    def start(self, wait_s: float = 300.0) -> "Fleet":
        for i, pl in enumerate(self.deployment.plan(self.first_gpu)):
            self.engines.append(self._spawn(pl, self.ports[i] if self.ports else self.base_port + i))
        self.wait_healthy(wait_s)
        return self

    def wait_healthy(self, wait_s: float = 300.0) -> None:
        deadline = time.time() + wait_s
        pending = list(self.engines)
        while pending:
            for e in list(pending):
                if not e.alive():
                    raise RuntimeError(f"engine on GPUs {e.placement.gpu_ids} exited with code {e.proc.returncode}")
                try:
                    with urllib.request.urlopen(e.url + "/health", timeout=2.0) as r:
                        if r.status == 200:
                            pending.remove(e)
                except Exception:
                    pass
            if pending:
                if time.time() > deadline:
                    raise TimeoutError(f"{len(pending)} engines did not come up within {wait_s:.0f} s")
                time.sleep(0.3)

    def start_router(self, port: int, model: Optional[str] = None, policy: str = "least_inflight", wait_s: float = 60.0,
                     failure_threshold: Optional[int] = None, timeout: Optional[float] = None,
                     max_connections: Optional[int] = None) -> str:
        """One router process in front of the engines of ``model`` (all engines if None); returns its URL. Generation
        requests go through it, weight updates still address the engines themselves."""
        cmd = [sys.executable, "-m", "miles_b200.router.router", "--port", str(port), "--policy", policy]
        for u in self.urls(model):
            cmd += ["--worker", u]
        for flag, v in (("--failure-threshold", failure_threshold), ("--timeout", timeout), ("--max-connections", max_connections)):
            if v is not None:
                cmd += [flag, str(v)]
        proc = subprocess.Popen(cmd, env=dict(os.environ, **self.env))
        self.__dict__.setdefault("routers", []).append(proc)
        url = f"http://127.0.0.1:{port}"
        deadline = time.time() + wait_s
        while True:
            if proc.poll() is not None:
                raise RuntimeError(f"the router exited with code {proc.returncode}")
            try:
                with urllib.request.urlopen(url + "/list_workers", timeout=2.0) as r:
                    if r.status == 200:
                        return url
            except Exception:
                pass
            if time.time() > deadline:
                raise TimeoutError("the router did not come up")
            time.sleep(0.2)

    def urls(self, model: Optional[str] = None, worker_type: Optional[str] = None) -> list:
        return [e.url for e in self.engines if (model is None or e.placement.model == model)
                and (worker_type is None or e.placement.worker_type == worker_type)]

    def updatable_urls(self) -> list:
        return [e.url for e in self.engines if e.placement.update_weights]

    def restart(self, index: int, wait_s: float = 300.0) -> EngineProcess:
        old = self.engines[index]
        if old.alive():
            old.proc.terminate()
            try:
                old.proc.wait(10)
            except subprocess.TimeoutExpired:
                old.proc.kill()
        self.engines[index] = self._spawn(old.placement, old.port)
        self.wait_healthy(wait_s)
        return self.engines[index]

    def monitor(self, interval: float = 10.0, timeout: float = 30.0, recover: bool = True, on_recovered=None):
        """A `ft.health.HealthMonitor` over the fleet: an engine that fails its probe is killed and, with ``recover``,
        replaced by a fresh process (``on_recovered(index, url)`` lets the caller reconnect it to the weight-update
        group and push the current weights)."""
        from ..ft.health import HealthMonitor

        mon: list = []

        def kill(i: int) -> None:
            e = self.engines[i]
            if e.alive():
                e.proc.kill()
            if recover:
                new = self.restart(i)
                mon[0].mark_recovered(i, new)
                if on_recovered is not None:
                    on_recovered(i, new.url)

        mon.append(HealthMonitor(self.engines, kill, interval=interval, timeout=timeout))
        return mon[0]

    def stop(self) -> None:
        for r in self.__dict__.get("routers", []):
            if r.poll() is None:
                r.terminate()
        for e in self.engines:
            if e.alive():
                e.proc.terminate()
        for e in self.engines:
            try:
                e.proc.wait(10)
            except subprocess.TimeoutExpired:
                e.proc.kill()
        self.engines = []
