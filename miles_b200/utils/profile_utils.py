"""Profiling hooks: torch profiler windows, CUDA memory history snapshots, periodic stack dumps.

``TrainProfiler`` implements ``--use-pytorch-profiler --profile-target {train_overall,train_actor,
train_log_probs} --profile-step-start/--profile-step-end`` (gzip TensorBoard traces per rank) and
``--record-memory-history --memory-snapshot-dir`` (snapshot dumped at the end of the window or on OOM).
Reference: miles/utils/profile_utils.py:13-147.  NVTX ranges (``nvtx_range``) wrap fused kernels' host call
sites so that external profilers show phase names.
"""
from __future__ import annotations

import contextlib
import faulthandler
import os
import sys
import threading

import torch


@contextlib.contextmanager
def nvtx_range(name: str):
    if torch.cuda.is_available():
        torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        yield


class TrainProfiler:
    def __init__(self, args, rank: int = 0):
        self.args, self.rank = args, rank
        self.enabled = bool(getattr(args, "use_pytorch_profiler", False))
        self.target = getattr(args, "profile_target", None) or "train_overall"
        self.start = getattr(args, "profile_step_start", 0) or 0
        self.end = getattr(args, "profile_step_end", self.start + 1) or (self.start + 1)
        self.dir = getattr(args, "tensorboard_dir", None) or getattr(args, "dump_details", None) or "profile_traces"
        self.prof = None
        self.mem_dir = getattr(args, "memory_snapshot_dir", None)
        if self.mem_dir and torch.cuda.is_available():
            torch.cuda.memory._record_memory_history(max_entries=100000)

    def step(self, rollout_id: int) -> None:
        if self.enabled and self.prof is None and rollout_id + 1 == self.start:
            acts = [torch.profiler.ProfilerActivity.CPU] + ([torch.profiler.ProfilerActivity.CUDA] if torch.cuda.is_available() else [])
            self.prof = torch.profiler.profile(activities=acts, record_shapes=True, with_stack=False, profile_memory=True)
            self.prof.start()
        elif self.prof is not None and rollout_id + 1 >= self.end:
            self.prof.stop()
            os.makedirs(self.dir, exist_ok=True)
            self.prof.export_chrome_trace(os.path.join(self.dir, f"trace_{self.target}_rank{self.rank}_step{rollout_id}.json.gz"))
            self.prof = None
        if self.mem_dir and torch.cuda.is_available() and rollout_id + 1 == (getattr(self.args, "memory_snapshot_num_steps", None) or 1):
            os.makedirs(self.mem_dir, exist_ok=True)
            torch.cuda.memory._dump_snapshot(os.path.join(self.mem_dir, f"memory_rank{self.rank}.pickle"))


class PeriodicStackDump:
    """Dumps the Python stacks of all threads every ``interval`` seconds (hang diagnosis without py-spy)."""

    def __init__(self, path: str, interval: float = 300.0):
        self.path, self.interval = path, interval
        self._stop = threading.Event()

    def start(self) -> None:
        def run():
            while not self._stop.wait(self.interval):
                with open(self.path, "a") as f:
                    faulthandler.dump_traceback(file=f, all_threads=True)

        threading.Thread(target=run, daemon=True).start()

    def stop(self) -> None:
        self._stop.set()


def print_memory(tag: str = "") -> dict:
    if not torch.cuda.is_available():
        return {}
    free, total = torch.cuda.mem_get_info()
    info = {"allocated_gb": torch.cuda.memory_allocated() / 1e9, "reserved_gb": torch.cuda.memory_reserved() / 1e9,
            "free_gb": free / 1e9, "total_gb": total / 1e9}
    print(f"[memory {tag}] " + " ".join(f"{k}={v:.2f}" for k, v in info.items()), file=sys.stderr)
    return info
