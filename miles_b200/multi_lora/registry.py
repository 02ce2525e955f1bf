"""Adapter slots and their life cycle.

``REGISTERED`` (declared through the API, no tensors yet) -> ``ACTIVE`` (tensors and optimizer exist, takes part in
rollout and training) -> ``DRAINING`` (deregistration requested: finishes the step it is in, is saved) ->
``REMOVED``. The number of live slots is bounded (``max_slots``); names are unique among live slots.
"""
from __future__ import annotations

import enum
import threading
from dataclasses import dataclass, field
from typing import Optional


class AdapterState(str, enum.Enum):
    REGISTERED = "registered"
    ACTIVE = "active"
    DRAINING = "draining"
    REMOVED = "removed"


@dataclass
class AdapterSpec:
    name: str
    rank: int = 16
    alpha: float = 32.0
    lr: float = 1e-4
    target_modules: object = "all-linear"
    rollout_batch_size: Optional[int] = None   # prompts per step for this adapter (None: the service default)
    prompt_data: Optional[str] = None          # its own dataset, if any (None: the service's --prompt-data)
    input_key: Optional[str] = None            # dataset columns of its own dataset (None: the service's)
    label_key: Optional[str] = None
    rm_type: Optional[str] = None              # its reward function (None: the service's --rm-type)
    num_step: Optional[int] = None             # retire (save + remove) after this many optimizer steps
    num_epoch: Optional[float] = None          # ... or after this many passes over its dataset (resolved to num_step)
    load: Optional[str] = None                 # PEFT directory to start from
    registration_id: str = ""                  # unique per registration: a re-registered name is a new tenant
    state: AdapterState = AdapterState.REGISTERED
    steps: int = 0
    slot: int = -1
    extra: dict = field(default_factory=dict)

    def to_dict(self) -> dict:
        d = dict(self.__dict__)
        d["state"] = self.state.value
        return d


class AdapterRegistry:
    def __init__(self, max_slots: int = 8, max_adapter_batch: Optional[int] = None, samples_per_prompt: int = 1):
        """``max_adapter_batch``: upper bound on an adapter's samples per optimizer step (its ``rollout_batch_size`` x
        ``samples_per_prompt``), checked when the adapter registers (``--multi-lora-max-adapter-global-batch-size``,
        default four times the global batch size)."""
        self.max_slots = max_slots
        self.max_adapter_batch, self.samples_per_prompt = max_adapter_batch, max(1, samples_per_prompt)
        self._lock = threading.Lock()
        self._adapters: dict = {}
        self.version = 0  # bumped on every change; the service loop compares it with its last snapshot

    def register(self, spec: AdapterSpec) -> AdapterSpec:
        with self._lock:
            live = [a for a in self._adapters.values() if a.state != AdapterState.REMOVED]
            if any(a.name == spec.name for a in live):
                raise ValueError(f"adapter {spec.name!r} is already registered")
            if len(live) >= self.max_slots:
                raise RuntimeError(f"all {self.max_slots} adapter slots are in use")
            if self.max_adapter_batch and spec.rollout_batch_size:
                n = spec.rollout_batch_size * self.samples_per_prompt
                if n > self.max_adapter_batch:
                    raise ValueError(f"adapter {spec.name!r} asks for {n} samples per step, more than the bound {self.max_adapter_batch}")
            used = {a.slot for a in live}
            spec.slot = next(i for i in range(self.max_slots) if i not in used)
            spec.state = AdapterState.REGISTERED
            import uuid

            spec.registration_id = uuid.uuid4().hex[:12]
            self._adapters[spec.name] = spec
            self.version += 1
            return spec

    def deregister(self, name: str) -> AdapterSpec:
        with self._lock:
            a = self._adapters.get(name)
            if a is None or a.state == AdapterState.REMOVED:
                raise KeyError(name)
            a.state = AdapterState.REMOVED if a.state == AdapterState.REGISTERED else AdapterState.DRAINING
            self.version += 1
            return a

    def transition(self, name: str, state: AdapterState) -> None:
        allowed = {AdapterState.REGISTERED: {AdapterState.ACTIVE, AdapterState.REMOVED},
                   AdapterState.ACTIVE: {AdapterState.DRAINING},
                   AdapterState.DRAINING: {AdapterState.REMOVED},
                   AdapterState.REMOVED: set()}
        with self._lock:
            a = self._adapters[name]
            if state not in allowed[a.state]:
                raise ValueError(f"adapter {name!r}: {a.state.value} -> {state.value} is not a valid transition")
            a.state = state
            self.version += 1

    def snapshot(self) -> tuple:
        """(version, [copies of the live specs in slot order])."""
        with self._lock:
            live = sorted((a for a in self._adapters.values() if a.state != AdapterState.REMOVED), key=lambda a: a.slot)
            return self.version, [AdapterSpec(**{**a.__dict__}) for a in live]

    def get(self, name: str) -> AdapterSpec:
        with self._lock:
            return self._adapters[name]

    def bump_steps(self, name: str) -> bool:
        """One more optimizer step trained. Returns True when the adapter has now reached its ``num_step`` (the caller
        deregisters it: it is saved and removed at the next reconciliation)."""
        with self._lock:
            a = self._adapters[name]
            a.steps += 1
            return a.num_step is not None and a.steps >= a.num_step

    def resolve_num_step(self, name: str, dataset_len: int, default_batch: int) -> Optional[int]:
        """``num_epoch`` -> ``num_step`` once the (filtered) dataset length is known."""
        with self._lock:
            a = self._adapters[name]
            if a.num_step is None and a.num_epoch is not None and dataset_len > 0:
                per = max(1, a.rollout_batch_size or default_batch)
                a.num_step = max(1, int(-(-a.num_epoch * dataset_len // per)))
            return a.num_step
