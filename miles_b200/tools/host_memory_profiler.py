"""Host-memory profiler: samples the machine's and this process's memory on a thread while the job runs, with phase marks
(rollout / train / weight update ...), writes a CSV, and summarises the peak per phase.

Why it exists here: optimizer state of large models lives partly in pinned host memory (trainer/optimizer.py), several
ranks share one host, and running out of host memory ends with the kernel's out-of-memory killer rather than an exception.
``--profile-host-memory out.csv`` turns it on in the training loop (rank 0 samples; the machine-wide numbers cover all
ranks).  ``python -m miles_b200.tools.host_memory_profiler out.csv`` prints the summary.

Reference: tools/cpu_memory_profiler.py (sampler + markers) and tools/visualize/cpu_memory_profiler_visualize.py (plots;
here a text summary).
"""
from __future__ import annotations

import csv
import os
import sys
import threading
import time
from typing import Optional


class HostMemoryProfiler:
    FIELDS = ("elapsed_s", "phase", "used_bytes", "available_bytes", "percent", "process_rss_bytes")

    def __init__(self, output_path: Optional[str] = None, interval: float = 0.5):
        self.output_path, self.interval = output_path, float(interval)
        self.records: list = []
        self.markers: list = []   # (elapsed_s, label)
        self._phase = "start"
        self._t0 = 0.0
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._lock = threading.Lock()

    def _sample(self) -> None:
        import psutil

        vm = psutil.virtual_memory()
        rss = psutil.Process(os.getpid()).memory_info().rss
        with self._lock:
            self.records.append((time.time() - self._t0, self._phase, int(vm.total - vm.available), int(vm.available),
                                 float(vm.percent), int(rss)))

    def _run(self) -> None:
        while not self._stop.wait(self.interval):
            self._sample()

    def start(self) -> "HostMemoryProfiler":
        self._t0 = time.time()
        self._stop.clear()
        self._sample()
        self._thread = threading.Thread(target=self._run, name="miles-b200-host-memory", daemon=True)
        self._thread.start()
        return self

    def mark(self, label: str) -> None:
        """Everything sampled from now on belongs to phase ``label``."""
        with self._lock:
            self._phase = str(label)
            self.markers.append((time.time() - self._t0, str(label)))
        self._sample()

    def stop(self) -> list:
        if self._thread is not None:
            self._stop.set()
            self._thread.join()
            self._thread = None
            self._sample()
        if self.output_path:
            self.write(self.output_path)
        return self.records

    def write(self, path: str) -> None:
        os.makedirs(os.path.dirname(os.path.abspath(path)) or ".", exist_ok=True)
        with open(path, "w", newline="") as f:
            w = csv.writer(f)
            w.writerow(self.FIELDS)
            with self._lock:
                w.writerows(self.records)


def summarize(path_or_records) -> list:
    """Per phase, in order of first appearance: ``{phase, seconds, samples, peak_used_gib, min_available_gib,
    peak_process_rss_gib}`` (phases named the same, e.g. every rollout, are pooled)."""
    if isinstance(path_or_records, str):
        with open(path_or_records) as f:
            rows = [(float(r["elapsed_s"]), r["phase"], int(r["used_bytes"]), int(r["available_bytes"]), float(r["percent"]),
                     int(r["process_rss_bytes"])) for r in csv.DictReader(f)]
    else:
        rows = list(path_or_records)
    out: dict = {}
    prev_t = rows[0][0] if rows else 0.0
    for t, phase, used, avail, _pct, rss in rows:
        s = out.setdefault(phase, {"phase": phase, "seconds": 0.0, "samples": 0, "peak_used_gib": 0.0,
                                   "min_available_gib": float("inf"), "peak_process_rss_gib": 0.0})
        s["seconds"] += max(t - prev_t, 0.0)
        prev_t = t
        s["samples"] += 1
        s["peak_used_gib"] = max(s["peak_used_gib"], used / 2**30)
        s["min_available_gib"] = min(s["min_available_gib"], avail / 2**30)
        s["peak_process_rss_gib"] = max(s["peak_process_rss_gib"], rss / 2**30)
    return list(out.values())


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if len(argv) != 1:
        print("usage: python -m miles_b200.tools.host_memory_profiler <profile.csv>")
        return 2
    print(f"{'phase':28s} {'seconds':>9s} {'peak used GiB':>14s} {'min avail GiB':>14s} {'peak RSS GiB':>13s}")
    for s in summarize(argv[0]):
        print(f"{s['phase']:28s} {s['seconds']:9.1f} {s['peak_used_gib']:14.2f} {s['min_available_gib']:14.2f} {s['peak_process_rss_gib']:13.2f}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
