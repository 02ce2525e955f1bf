"""Collects what the dashboard shows: step metrics (a tracking sink), trajectory life-cycle events (a lifecycle
sink) and periodic GPU samples (utilisation, memory, power, SM clock through NVML; read-only)."""
from __future__ import annotations

import threading
from typing import Callable, Optional

from .store import EventStore


def _nvml_sampler() -> Optional[Callable[[], list]]:
    try:
        import pynvml

        pynvml.nvmlInit()
        n = pynvml.nvmlDeviceGetCount()
        handles = [pynvml.nvmlDeviceGetHandleByIndex(i) for i in range(n)]
    except Exception:  # noqa: BLE001 - no driver on this host
        return None

    def sample() -> list:
        out = []
        for i, h in enumerate(handles):
            try:
                u = pynvml.nvmlDeviceGetUtilizationRates(h)
                m = pynvml.nvmlDeviceGetMemoryInfo(h)
                out.append({"gpu": i, "util": u.gpu, "mem_used": m.used, "mem_total": m.total,
                            "power_w": pynvml.nvmlDeviceGetPowerUsage(h) / 1000.0,
                            "sm_mhz": pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)})
            except Exception:  # noqa: BLE001
                continue
        return out

    return sample


class Collector:
    def __init__(self, store: EventStore, gpu_interval: float = 5.0, gpu_sampler: Optional[Callable[[], list]] = None,
                 engine_interval: Optional[float] = None, engine_metrics: Optional[list] = None, forward: Optional[Callable] = None):
        """``engine_interval``: scrape cadence of the engines' ``/metrics`` (default: with every GPU sample);
        ``engine_metrics``: keep only these metric names of an engine's answer; ``forward(name, value, labels)``: also hand
        every gauge to another sink (the Prometheus backend)."""
        self.store = store
        self.gpu_interval = gpu_interval
        self.engine_interval = engine_interval
        self.engine_metrics = set(engine_metrics) if engine_metrics else None
        self.forward = forward
        self._sampler = gpu_sampler if gpu_sampler is not None else _nvml_sampler()
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None

    # sinks -----------------------------------------------------------------------------------------------
    def log_metrics(self, metrics: dict, step: int) -> None:
        self.store.append("metrics", {"step": step, **{k: v for k, v in metrics.items() if isinstance(v, (int, float))}})

    def on_lifecycle(self, rec: dict) -> None:
        self.store.append("trajectories", rec, t=rec.get("t"))

    def sample_gpus_once(self) -> int:
        if self._sampler is None:
            return 0
        rows = self._sampler()
        for r in rows:
            self.store.append("gpus", r)
            if self.forward is not None:
                for k, v in r.items():
                    if isinstance(v, (int, float)) and k not in ("gpu", "index"):
                        self.forward(f"dashboard_gpu_{k}", float(v), {"gpu": str(r.get("gpu", r.get("index", "")))})
        return len(rows)

    def add_engine(self, url: str) -> None:
        """Scrape this engine's ``/metrics`` (Prometheus text) with every sampling tick."""
        self.__dict__.setdefault("_engines", []).append(url.rstrip("/"))

    def scrape_engines_once(self, fetch: Optional[Callable[[str], str]] = None) -> int:
        n = 0
        for url in self.__dict__.get("_engines", []):
            try:
                text = fetch(url + "/metrics") if fetch is not None else _http_get(url + "/metrics")
            except Exception as e:  # an engine that does not answer is itself a data point
                self.store.append("engines", {"engine": url, "up": 0, "error": repr(e)[:120]})
                continue
            rec = {"engine": url, "up": 1}
            vals = parse_prometheus(text)
            if self.engine_metrics is not None:
                vals = {k: v for k, v in vals.items() if k in self.engine_metrics}
            rec.update(vals)
            self.store.append("engines", rec)
            if self.forward is not None:
                for k, v in vals.items():
                    self.forward(f"dashboard_engine_{k}", float(v), {"engine": url})
            n += 1
        return n

    # background sampling ---------------------------------------------------------------------------------
    def start(self) -> None:
        if (self._sampler is None and not self.__dict__.get("_engines")) or self._thread is not None:
            return

        def loop():
            import time

            step = min(self.gpu_interval, self.engine_interval or self.gpu_interval)
            next_gpu = next_eng = time.monotonic()
            while not self._stop.wait(step):
                now = time.monotonic()
                if now >= next_gpu:
                    self.sample_gpus_once()
                    next_gpu = now + self.gpu_interval
                if now >= next_eng:
                    self.scrape_engines_once()
                    next_eng = now + (self.engine_interval or self.gpu_interval)

        self._thread = threading.Thread(target=loop, daemon=True)
        self._thread.start()

    def stop(self) -> None:
        self._stop.set()


def _http_get(url: str, timeout: float = 2.0) -> str:
    import urllib.request

    with urllib.request.urlopen(url, timeout=timeout) as r:
        return r.read().decode()


def parse_prometheus(text: str) -> dict:
    """``name{labels} value`` lines -> {name: value} (labels dropped, comments skipped, last sample wins)."""
    out = {}
    for line in text.splitlines():
        line = line.strip()
        if not line or line.startswith("#"):
            continue
        parts = line.rsplit(" ", 1)
        if len(parts) != 2:
            continue
        name = parts[0].split("{", 1)[0].strip()
        try:
            out[name] = float(parts[1])
        except ValueError:
            continue
    return out


def advisories(store: EventStore, window: int = 20) -> list:
    """Plain-language hints from the recent history (each rule is a few lines: easy to read, easy to extend)."""
    out = []
    ms = store.tail("metrics", window)
    if ms:
        last = ms[-1]
        ro, tr = last.get("perf/rollout_time"), last.get("perf/train_time")
        if ro and tr and ro > 3 * tr:
            out.append({"rule": "rollout_bound", "text": f"rollout takes {ro:.1f}s against {tr:.1f}s of training: "
                        "consider the fully-asynchronous driver or a larger rollout batch per GPU"})
        d = last.get("train/train_rollout_logprob_abs_diff")
        if d is not None and d > 0.05:
            out.append({"rule": "train_rollout_mismatch", "text": f"trainer/rollout log-prob difference {d:.3f} is high: "
                        "check routing replay (MoE) and importance-sampling correction"})
        trunc = last.get("rollout/truncated_ratio")
        if trunc is not None and trunc > 0.3:
            out.append({"rule": "truncation", "text": f"{trunc:.0%} of the responses hit the length limit"})
        norms = [m.get("train/grad_norm") for m in ms if m.get("train/grad_norm") is not None]
        if len(norms) >= 5 and norms[-1] > 10 * (sum(norms[:-1]) / len(norms[:-1]) + 1e-9):
            out.append({"rule": "grad_spike", "text": f"gradient norm {norms[-1]:.2f} is more than 10x its recent mean"})
    es = store.tail("engines", 16)
    down = sorted({e["engine"] for e in es[-4:] if not e.get("up")})
    if down:
        out.append({"rule": "engine_down", "text": "no answer from " + ", ".join(down)})
    queued = [e for e in es[-4:] if e.get("miles_b200:num_queue_reqs", 0) > 4 * max(e.get("miles_b200:num_running_reqs", 0), 1)]
    if queued:
        out.append({"rule": "engine_queue", "text": f"{queued[-1]['engine']} queues {int(queued[-1]['miles_b200:num_queue_reqs'])} requests: "
                    "raise --sglang-max-running-requests or add engines"})
    gs = store.tail("gpus", 64)
    low = [g for g in gs if g.get("sm_mhz") and g.get("util", 0) > 80 and g["sm_mhz"] < 1000]
    if low:
        out.append({"rule": "low_clocks", "text": f"GPU {low[-1]['gpu']} runs at {low[-1]['sm_mhz']} MHz under load"})
    return out
