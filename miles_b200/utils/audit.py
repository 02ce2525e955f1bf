"""Audit trail: typed events, the witness table and analyzer rules.

* ``EventLogger``: append-only JSONL of events stamped with process identity and a per-process sequence number; the
  position survives a resume (``state_dict`` / ``load_state_dict``). Events are plain dicts with a ``kind``; the
  constructors below (``ev_*``) fix each kind's fields.
* ``WitnessAllocator`` + ``Witness``: every sample of a rollout gets a slot of a small ring table. Training a sample adds
  one to its slot through the same commit / discard boundary as the optimizer step, and the table is *read back* into
  the event log after the step, so what the analyzer sees is what the table holds, not what the caller believes.
  When the ring wraps, the slots it hands out again are cleared and listed as stale so that old counts are not
  mistaken for new ones.
* Analyzer rules (``RULES``): all replicas report the same weight checksum per step; every engine reports the trainer's
  checksum after a sync; for every rollout whose steps all ended normally each allocated slot reads exactly 1 (no
  sample skipped, none trained twice across retries and healed cells), and a rollout with a discarded step left no count
  behind for the samples of that step.

Reference: miles/utils/audit_utils/{event_logger,event_analyzer/rules,witness}/*.
"""
from __future__ import annotations

import json
import os
import socket
import time
from collections import defaultdict
from typing import Callable, Iterable, Optional

import torch

# ---------------------------------------------------------------------------------------------- events
KINDS = ("train_step", "weight_checksum", "engine_checksum", "witness_allocate", "witness", "cell_state", "weight_update")


def process_identity(role: str = "", rank: int = 0) -> dict:
    return {"host": socket.gethostname(), "pid": os.getpid(), "role": role, "rank": rank}


def ev_train_step(rollout_id: int, step: int, samples: int, outcome: str = "normal", sample_indices: Optional[list] = None) -> dict:
    assert outcome in ("normal", "discarded")
    return {"kind": "train_step", "rollout_id": int(rollout_id), "step": int(step), "samples": int(samples), "outcome": outcome,
            "sample_indices": [int(i) for i in (sample_indices or [])]}


def ev_weight_checksum(step: int, version: int, checksum: str) -> dict:
    return {"kind": "weight_checksum", "step": int(step), "version": int(version), "checksum": str(checksum)}


def ev_engine_checksum(engine: str, version: int, checksum: str) -> dict:
    return {"kind": "engine_checksum", "engine": str(engine), "version": int(version), "checksum": str(checksum)}


def ev_witness_allocate(rollout_id: int, sample_indices: list, witness_ids: list, stale_ids: list) -> dict:
    return {"kind": "witness_allocate", "rollout_id": int(rollout_id), "sample_indices": [int(i) for i in sample_indices],
            "witness_ids": [int(i) for i in witness_ids], "stale_ids": [int(i) for i in stale_ids]}


def ev_witness_snapshot(rollout_id: int, step: int, counts: dict) -> dict:
    """``counts``: witness id -> what the table holds after the step (read back from the table)."""
    return {"kind": "witness", "rollout_id": int(rollout_id), "step": int(step), "counts": {str(k): int(v) for k, v in counts.items()}}


class EventLogger:
    def __init__(self, directory: Optional[str], role: str = "", rank: int = 0):
        self.path = None
        self.identity = process_identity(role, rank)
        self.events: list = []
        self.seq = 0
        if directory:
            os.makedirs(directory, exist_ok=True)
            self.path = os.path.join(directory, f"events-{role or 'proc'}-{rank:05d}.jsonl")

    def log(self, kind, **fields) -> dict:
        """``log("kind", field=...)`` or ``log(event_dict)`` (from an ``ev_*`` constructor)."""
        if isinstance(kind, dict):
            fields, kind = {k: v for k, v in kind.items() if k != "kind"}, kind["kind"]
        ev = {"kind": kind, "ts": time.time(), "seq": self.seq, **self.identity, **fields}
        self.seq += 1
        self.events.append(ev)
        if self.path:
            with open(self.path, "a") as f:
                f.write(json.dumps(ev, default=str) + "\n")
        return ev

    def state_dict(self) -> dict:
        return {"seq": self.seq}

    def load_state_dict(self, sd: dict) -> None:
        """After a resume the sequence continues where the checkpoint left it (events of the lost steps stay in the
        file: the analyzer orders by (pid, seq) within a process and by time across processes)."""
        self.seq = max(self.seq, int(sd.get("seq", 0)))


def read_events(directory: str) -> list:
    out = []
    for fn in sorted(os.listdir(directory)):
        if fn.startswith("events-") and fn.endswith(".jsonl"):
            with open(os.path.join(directory, fn)) as f:
                out += [json.loads(l) for l in f if l.strip()]
    return sorted(out, key=lambda e: (e["ts"], e.get("seq", 0)))


# ---------------------------------------------------------------------------------------------- witness
class WitnessAllocator:
    """Hands out slots of a ring of ``size`` witness ids. ``allocate`` returns ``(witness_ids, stale_ids)``: the slots for
    the given samples and, among them, the ones that had an earlier owner (whose counts the caller must clear)."""

    def __init__(self, size: int):
        self.size = int(size)
        self.next = 0
        self.owner: dict = {}        # witness id -> (rollout_id, sample_index)
        self.by_sample: dict = {}    # (rollout_id, sample_index) -> witness id

    def allocate(self, rollout_id: int, sample_indices: Iterable[int]) -> tuple:
        wids, stale = [], []
        for s in sample_indices:
            key = (int(rollout_id), int(s))
            if key in self.by_sample:        # the same rollout staged again (a retried step): same slot
                wids.append(self.by_sample[key])
                continue
            w = self.next
            self.next = (self.next + 1) % self.size
            old = self.owner.get(w)
            if old is not None:
                stale.append(w)
                self.by_sample.pop(old, None)
            self.owner[w] = key
            self.by_sample[key] = w
            wids.append(w)
        return wids, stale

    def state_dict(self) -> dict:
        return {"next": self.next, "owner": {str(k): list(v) for k, v in self.owner.items()}}

    def load_state_dict(self, sd: dict) -> None:
        self.next = int(sd.get("next", 0))
        self.owner = {int(k): (int(v[0]), int(v[1])) for k, v in sd.get("owner", {}).items()}
        self.by_sample = {v: k for k, v in self.owner.items()}


class Witness:
    def __init__(self, size: int, device="cpu"):
        self.size = size
        self.table = torch.zeros(size, dtype=torch.int64, device=device)
        self.pending = torch.zeros_like(self.table)
        self.allocator = WitnessAllocator(size)

    def allocate(self, rollout_id: int, sample_indices: Iterable[int]) -> tuple:
        """Slots for a rollout's samples; slots that the ring reuses are cleared first. Returns (witness ids, stale ids)."""
        wids, stale = self.allocator.allocate(rollout_id, sample_indices)
        if stale:
            idx = torch.as_tensor(stale, dtype=torch.int64, device=self.table.device)
            self.table[idx] = 0
            self.pending[idx] = 0
        return wids, stale

    def touch(self, witness_ids: Iterable[int]) -> None:
        ids = torch.as_tensor([int(i) % self.size for i in witness_ids], dtype=torch.int64, device=self.table.device)
        if ids.numel():
            self.pending.index_add_(0, ids, torch.ones_like(ids))

    def commit(self) -> None:
        """Called together with the optimizer step: a discarded step calls ``discard`` instead."""
        self.table += self.pending
        self.pending.zero_()

    def discard(self) -> None:
        self.pending.zero_()

    def counts(self, witness_ids: Iterable[int]) -> dict:
        return {int(i): int(self.table[int(i) % self.size]) for i in witness_ids}

    def reset(self) -> None:
        self.table.zero_()
        self.pending.zero_()

    def state_dict(self) -> dict:
        return {"table": self.table.clone(), "allocator": self.allocator.state_dict()}

    def load_state_dict(self, sd: dict) -> None:
        self.table.copy_(sd["table"])
        self.pending.zero_()
        self.allocator.load_state_dict(sd.get("allocator", {}))


# ---------------------------------------------------------------------------------------------- analyzer rules
def rule_cross_replica_weight_checksum(events: list) -> list:
    by_step = defaultdict(set)
    for e in events:
        if e["kind"] == "weight_checksum":
            by_step[e["step"]].add(e["checksum"])
    return [f"replicas disagree on the weight checksum at step {step}: {sorted(cks)}" for step, cks in sorted(by_step.items()) if len(cks) > 1]


def rule_engine_checksum_consistency(events: list) -> list:
    trainer = {}
    for e in events:
        if e["kind"] == "weight_checksum":
            trainer[e.get("version", e["step"])] = e["checksum"]
    out = []
    for e in events:
        if e["kind"] == "engine_checksum":
            want = trainer.get(e["version"])
            if want is not None and want != e["checksum"]:
                out.append(f"engine {e.get('engine')} holds checksum {e['checksum']} for version {e['version']}, trainer has {want}")
    return out


def rule_witness_exactly_once(events: list) -> list:
    """Per trainer process: after the last snapshot of a rollout, every slot allocated to it reads 1 if all its steps ended
    normally; samples of a discarded step read 0. Slots the ring has since handed to a later rollout are skipped."""
    out = []
    procs = defaultdict(list)
    for e in events:
        procs[(e.get("host"), e.get("pid"), e.get("role"), e.get("rank"))].append(e)
    for ident, evs in procs.items():
        alloc: dict = {}     # rollout -> {sample_index: witness id}
        stale_after: dict = defaultdict(set)
        discarded: dict = defaultdict(set)   # rollout -> sample indices of discarded steps
        trained: dict = defaultdict(set)     # rollout -> sample indices of normal steps
        last: dict = {}      # rollout -> counts of its last snapshot
        for e in evs:
            k = e["kind"]
            if k == "witness_allocate":
                m = alloc.setdefault(e["rollout_id"], {})
                m.update(dict(zip(e["sample_indices"], e["witness_ids"])))
                for r in alloc:
                    if r != e["rollout_id"]:
                        stale_after[r].update(w for w in e["stale_ids"])
            elif k == "train_step":
                (discarded if e.get("outcome") == "discarded" else trained)[e["rollout_id"]].update(e.get("sample_indices", []))
            elif k == "witness":
                last.setdefault(e["rollout_id"], {}).update({int(w): c for w, c in e["counts"].items()})
        for rid, m in alloc.items():
            if rid not in last:
                if trained.get(rid):
                    out.append(f"{ident}: rollout {rid} trained {len(trained[rid])} samples but left no witness snapshot")
                continue
            for s, w in m.items():
                if w in stale_after[rid]:
                    continue
                c = last[rid].get(w)
                want = 1 if s in trained.get(rid, ()) else 0
                if s in discarded.get(rid, ()) and s not in trained.get(rid, ()):
                    want = 0
                if c is None:
                    if want:
                        out.append(f"{ident}: sample {s} of rollout {rid} (witness {w}) is missing from the snapshot")
                elif c != want:
                    out.append(f"{ident}: sample {s} of rollout {rid} was trained {c} times, expected {want}")
    return out


RULES: dict = {"cross_replica_weight_checksum": rule_cross_replica_weight_checksum,
               "engine_checksum_consistency": rule_engine_checksum_consistency,
               "witness_exactly_once": rule_witness_exactly_once}


def analyze(events: Iterable[dict], rules: Optional[Iterable[str]] = None) -> list:
    """Returns the violations found by the chosen rules (all by default); empty = consistent."""
    evs = list(events)
    problems = []
    for name in (rules or RULES):
        fn: Callable = RULES[name]
        problems += fn(evs)
    return problems
