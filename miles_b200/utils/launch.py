"""Launch helpers: build the ``torchrun`` command line of a training job from a typed description, the environment
it needs on an NVLink box, and run checkpoint conversions — the role of the reference's
``execute_train`` / ``convert_checkpoint`` / NVLink detection (miles/utils/external_utils/command_utils.py:104-233),
without Ray: one process per GPU on one node.
"""
from __future__ import annotations

import os
import shlex
import subprocess
import sys
from dataclasses import dataclass, field
from typing import Optional, Sequence


@dataclass
class TrainJob:
    script: str = "train.py"
    num_gpus: int = 8
    args: Sequence[str] = field(default_factory=list)
    master_addr: str = "127.0.0.1"
    master_port: int = 29500
    env: dict = field(default_factory=dict)

    def command(self) -> list:
        return [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={self.num_gpus}",
                "--master-addr", self.master_addr, "--master-port", str(self.master_port), self.script, *self.args]

    def environment(self, base: Optional[dict] = None) -> dict:
        env = dict(os.environ if base is None else base)
        env.setdefault("CUDA_DEVICE_MAX_CONNECTIONS", "1")
        env.setdefault("NCCL_NVLS_ENABLE", "1" if has_nvlink() else "0")
        env.setdefault("PYTHONUNBUFFERED", "1")
        env.update({k: str(v) for k, v in self.env.items()})
        return env

    def shell_line(self) -> str:
        return " ".join(shlex.quote(c) for c in self.command())


def has_nvlink() -> bool:
    """Whether GPU 0 reports an active NVLink (read through NVML; False when there is no GPU or no NVML)."""
    try:
        import pynvml

        pynvml.nvmlInit()
        try:
            h = pynvml.nvmlDeviceGetHandleByIndex(0)
            for link in range(18):
                try:
                    if pynvml.nvmlDeviceGetNvLinkState(h, link):
                        return True
                except pynvml.NVMLError:
                    break
            return False
        finally:
            pynvml.nvmlShutdown()
    except Exception:
        return False


def execute_train(job: TrainJob, dry_run: bool = False, log_path: Optional[str] = None) -> int:
    """Run the job and wait for it; returns its exit code (``dry_run`` only prints the command)."""
    if dry_run:
        print(job.shell_line())
        return 0
    out = open(log_path, "ab") if log_path else None
    try:
        return subprocess.run(job.command(), env=job.environment(), stdout=out, stderr=subprocess.STDOUT if out else None).returncode
    finally:
        if out:
            out.close()


def convert_checkpoint(src: str, dst: str, direction: str = "hf_to_native", expert_parallel: int = 1,
                       dry_run: bool = False) -> int:
    """Run one of the converters in ``miles_b200.tools`` as a child process."""
    if direction == "hf_to_native":
        cmd = [sys.executable, "-m", "miles_b200.tools.convert_hf_to_native", "--hf-checkpoint", src, "--save", dst]
    elif direction == "native_to_hf":
        cmd = [sys.executable, "-m", "miles_b200.tools.convert_native_to_hf", "--load", src, "--output", dst]
    else:
        raise ValueError(f"unknown direction {direction!r}")
    if direction == "hf_to_native" and expert_parallel > 1:
        cmd += ["--expert-model-parallel-size", str(expert_parallel)]
    if dry_run:
        print(" ".join(shlex.quote(c) for c in cmd))
        return 0
    return subprocess.run(cmd).returncode
