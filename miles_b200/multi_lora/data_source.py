"""Per-adapter prompt streams of the multi-LoRA service.

Every adapter trains on its own data: its own prompt file (or the service's), its own reward function, its own batch
size. ``AdapterDataSources`` keeps one data source per live adapter (built from a copy of the service's arguments with
the adapter's overrides, seeded per slot), stamps every sample it hands out with the adapter's name, registration id
and reward type, and drops the source of an adapter that is gone.

Reference: miles/rollout/multi_lora/data_source.py:31-137.
"""
from __future__ import annotations

import copy
from typing import Callable, Optional

from .registry import AdapterRegistry, AdapterSpec


class _Stamped:
    """A data source whose samples carry their adapter (so reward dispatch, logging and training know whose they are)."""

    def __init__(self, inner, spec: AdapterSpec):
        self.inner, self.name, self.registration_id, self.rm_type = inner, spec.name, spec.registration_id, spec.rm_type

    def get_samples(self, num_samples: int) -> list:
        groups = self.inner.get_samples(num_samples)
        for g in groups:
            for s in g:
                md = dict(s.metadata or {}, adapter=self.name, adapter_registration=self.registration_id)
                if self.rm_type:
                    md["rm_type"] = self.rm_type   # the reward hub looks here before --rm-type
                s.metadata = md
        return groups

    def __getattr__(self, item):
        return getattr(self.inner, item)


class AdapterDataSources:
    def __init__(self, args, tokenizer, build: Callable, registry: Optional[AdapterRegistry] = None, default_batch: int = 1):
        """``build(args, tokenizer) -> data source`` (the loop's own constructor, so buffers / synthetic sources work)."""
        self.args, self.tokenizer, self.build, self.registry, self.default_batch = args, tokenizer, build, registry, default_batch
        self.sources: dict = {}

    def _args_for(self, spec: AdapterSpec):
        a = copy.copy(self.args)
        for key in ("prompt_data", "input_key", "label_key"):
            v = getattr(spec, key)
            if v is not None:
                setattr(a, key, v)
        a.rollout_seed = getattr(self.args, "rollout_seed", 0) + 104729 * (spec.slot + 1)   # adapters draw different streams
        return a

    def reconcile(self, specs: list) -> None:
        live = {s.name: s for s in specs}
        for name in list(self.sources):
            if name not in live or self.sources[name].registration_id != live[name].registration_id:
                del self.sources[name]    # gone, or the name was registered again: a new tenant starts from its first prompt
        for name, spec in live.items():
            if name not in self.sources:
                src = self.build(self._args_for(spec), self.tokenizer)
                self.sources[name] = _Stamped(src, spec)
                ds = getattr(src, "dataset", None)
                if self.registry is not None and ds is not None:
                    self.registry.resolve_num_step(name, len(ds), self.default_batch)

    def get(self, name: str) -> _Stamped:
        return self.sources[name]
