"""Audit trail: event log, analyzer rules and the witness parameter.

* ``EventLogger``: append-only JSONL of typed events (``train_step``, ``weight_checksum``, ``engine_checksum``,
  ``cell_state``, ``witness``...) stamped with process identity.
* ``analyze``: rules over an event stream — all replicas report the same weight checksum per step, every
  engine reports the trainer's checksum after a sync, witness counts are exactly one per sample.
* ``Witness``: a tiny embedding-like table with one row per sample-id slot; training a sample adds 1 to its
  row through the same optimizer-step boundary as the real update, so after retries / healed cells each
  sample id must have been counted exactly once (proves exactly-once training).
Reference: miles/utils/audit_utils/* (event_logger, event_analyzer/rules, witness.py).
"""
from __future__ import annotations

import json
import os
import socket
import time
from collections import defaultdict
from typing import Iterable, Optional

import torch


def process_identity(role: str = "", rank: int = 0) -> dict:
    return {"host": socket.gethostname(), "pid": os.getpid(), "role": role, "rank": rank}


class EventLogger:
    def __init__(self, directory: Optional[str], role: str = "", rank: int = 0):
        self.path = None
        self.identity = process_identity(role, rank)
        self.events: list = []
        if directory:
            os.makedirs(directory, exist_ok=True)
            self.path = os.path.join(directory, f"events-{role or 'proc'}-{rank:05d}.jsonl")

    def log(self, kind: str, **fields) -> dict:
        ev = {"kind": kind, "ts": time.time(), **self.identity, **fields}
        self.events.append(ev)
        if self.path:
            with open(self.path, "a") as f:
                f.write(json.dumps(ev, default=str) + "\n")
        return ev


def read_events(directory: str) -> list:
    out = []
    for fn in sorted(os.listdir(directory)):
        if fn.startswith("events-") and fn.endswith(".jsonl"):
            with open(os.path.join(directory, fn)) as f:
                out += [json.loads(l) for l in f if l.strip()]
    return sorted(out, key=lambda e: e["ts"])


def analyze(events: Iterable[dict]) -> list:
    """Returns a list of violations (empty = consistent)."""
    problems = []
    by_step = defaultdict(set)
    trainer_ck = {}
    for e in events:
        if e["kind"] == "weight_checksum":
            by_step[e["step"]].add(e["checksum"])
            trainer_ck[e.get("version", e["step"])] = e["checksum"]
    for step, cks in by_step.items():
        if len(cks) > 1:
            problems.append(f"replicas disagree on the weight checksum at step {step}: {sorted(cks)}")
    for e in events:
        if e["kind"] == "engine_checksum":
            want = trainer_ck.get(e["version"])
            if want is not None and want != e["checksum"]:
                problems.append(f"engine {e.get('engine')} holds checksum {e['checksum']} for version {e['version']}, trainer has {want}")
    counts = defaultdict(int)
    for e in events:
        if e["kind"] == "witness":
            for sid, c in e["counts"].items():
                counts[(e["rollout_id"], sid)] += c
    for (rid, sid), c in counts.items():
        if c != 1:
            problems.append(f"sample {sid} of rollout {rid} was trained {c} times")
    return problems


class Witness:
    def __init__(self, size: int, device="cpu"):
        self.size = size
        self.table = torch.zeros(size, dtype=torch.int64, device=device)
        self.pending = torch.zeros_like(self.table)

    def touch(self, sample_ids: Iterable[int]) -> None:
        ids = torch.as_tensor(list(sample_ids), dtype=torch.int64, device=self.table.device) % self.size
        self.pending.index_add_(0, ids, torch.ones_like(ids))

    def commit(self) -> None:
        """Called together with the optimizer step: a discarded step calls ``discard`` instead."""
        self.table += self.pending
        self.pending.zero_()

    def discard(self) -> None:
        self.pending.zero_()

    def counts(self, sample_ids: Iterable[int]) -> dict:
        return {int(i): int(self.table[int(i) % self.size]) for i in sample_ids}

    def reset(self) -> None:
        self.table.zero_()
        self.pending.zero_()
