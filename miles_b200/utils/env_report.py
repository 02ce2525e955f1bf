"""Environment report of a node: library versions, GPUs, driver, the environment variables that steer collectives
and the git state of the source tree — printed at start-up and attached to the run's metadata so that two runs can
be compared after the fact. Encoded as one marked JSON line so that a launcher can fish it out of a worker's log.

Reference counterpart: miles/utils/env_report.py:13-200.
"""
from __future__ import annotations

import json
import os
import platform
import socket
import subprocess
import sys
from dataclasses import asdict, dataclass, field
from typing import Optional

MARK = "MILES_B200_ENV_REPORT "
ENV_PREFIXES = ("NCCL_", "CUDA_", "TORCH_", "MILES_", "OMP_", "MASTER_", "WORLD_SIZE", "RANK", "LOCAL_RANK")


@dataclass
class GitInfo:
    root: str
    commit: Optional[str] = None
    dirty: Optional[bool] = None
    branch: Optional[str] = None


@dataclass
class NodeEnvReport:
    hostname: str
    python: str
    platform: str
    packages: dict = field(default_factory=dict)
    cuda: dict = field(default_factory=dict)
    gpus: list = field(default_factory=list)
    env: dict = field(default_factory=dict)
    git: Optional[GitInfo] = None


def _git(root: str) -> Optional[GitInfo]:
    def run(*a):
        try:
            r = subprocess.run(["git", "-C", root, *a], capture_output=True, text=True, timeout=5)
            return r.stdout.strip() if r.returncode == 0 else None
        except Exception:
            return None

    commit = run("rev-parse", "HEAD")
    if commit is None:
        return None
    status = run("status", "--porcelain")
    return GitInfo(root, commit, bool(status) if status is not None else None, run("rev-parse", "--abbrev-ref", "HEAD"))


def collect(packages=("torch", "numpy", "transformers", "flash_attn", "safetensors", "pydantic", "fastapi")) -> NodeEnvReport:
    import importlib

    rep = NodeEnvReport(socket.gethostname(), sys.version.split()[0], platform.platform())
    from importlib import metadata

    for p in packages:
        try:  # the installed version from the package metadata: nothing is imported for the report
            rep.packages[p] = metadata.version(p.replace("_", "-"))
        except Exception:
            mod = sys.modules.get(p)
            rep.packages[p] = getattr(mod, "__version__", None) if mod is not None else None
    try:
        import torch

        rep.cuda = {"torch_cuda": torch.version.cuda, "available": torch.cuda.is_available(),
                    "nccl": ".".join(map(str, torch.cuda.nccl.version())) if torch.cuda.is_available() else None}
        if torch.cuda.is_available():
            for i in range(torch.cuda.device_count()):
                pr = torch.cuda.get_device_properties(i)
                rep.gpus.append({"index": i, "name": pr.name, "memory_gib": round(pr.total_memory / 2**30, 1),
                                 "sms": pr.multi_processor_count, "capability": f"{pr.major}.{pr.minor}"})
    except Exception as e:  # a report must never take the job down
        rep.cuda = {"error": repr(e)}
    try:
        import pynvml

        pynvml.nvmlInit()
        rep.cuda["driver"] = pynvml.nvmlSystemGetDriverVersion()
        pynvml.nvmlShutdown()
    except Exception:
        pass
    rep.env = {k: v for k, v in sorted(os.environ.items()) if k.startswith(ENV_PREFIXES)}
    rep.git = _git(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
    return rep


def encode(rep: NodeEnvReport) -> str:
    return MARK + json.dumps(asdict(rep), sort_keys=True)


def decode(line: str) -> Optional[dict]:
    """The report found in a log line (anywhere in it), or None."""
    i = line.find(MARK)
    if i < 0:
        return None
    try:
        return json.loads(line[i + len(MARK):])
    except json.JSONDecodeError:
        return None


def collect_and_print(stream=None) -> NodeEnvReport:
    rep = collect()
    print(encode(rep), file=stream or sys.stderr, flush=True)
    return rep


def diff(a: dict, b: dict, prefix: str = "") -> list:
    """Keys whose values differ between two decoded reports (dotted paths)."""
    out: list = []
    for k in sorted(set(a) | set(b)):
        va, vb = a.get(k), b.get(k)
        if isinstance(va, dict) and isinstance(vb, dict):
            out += diff(va, vb, f"{prefix}{k}.")
        elif va != vb:
            out.append((f"{prefix}{k}", va, vb))
    return out
