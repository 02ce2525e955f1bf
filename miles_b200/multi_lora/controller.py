"""Reconciles the registry with the adapters that actually exist on the trainer, and exposes the HTTP control API.

One base model serves every adapter. Adapters are kept in merged form (see ``miles_b200/lora.py``): activating an
adapter writes ``W_base + scale * B A`` into the live weights, which the colocated engine shares, so rollout and
training of the active adapter need no further hand-off; switching adapters costs one merge. Each slot owns its
adapter tensors and its optimizer, so gradient history is kept per adapter across steps.
"""

import os
from typing import Callable, Optional

from ..lora import LoRAManager
from .registry import AdapterRegistry, AdapterSpec, AdapterState


class MultiLoRAController:
    def __init__(self, actor, registry: Optional[AdapterRegistry] = None, save_dir: Optional[str] = None):
        self.actor = actor
        self.registry = registry or AdapterRegistry()
        self.save_dir = save_dir
        self.managers: dict = {}   # name -> LoRAManager
        self.base: dict = {}       # native name -> frozen base tensor, shared by all adapters
        self.active: Optional[str] = None
        self._seen_version = -1

    # ------------------------------------------------------------------ reconciliation
    def reconcile(self) -> list:
        """Create tensors for newly registered adapters, save and drop draining ones. Returns the names that are
        ACTIVE afterwards (slot order)."""
        version, specs = self.registry.snapshot()
        for a in specs:
            if a.state == AdapterState.REGISTERED:
                self._create(a)
                self.registry.transition(a.name, AdapterState.ACTIVE)
            elif a.state == AdapterState.DRAINING:
                self._retire(a)
                self.registry.transition(a.name, AdapterState.REMOVED)
        self._seen_version = version
        return [a.name for a in self.registry.snapshot()[1] if a.state == AdapterState.ACTIVE]

    def _create(self, a: AdapterSpec) -> None:
        base = self._base_store()
        m = LoRAManager(base, a.rank, a.alpha, a.target_modules, lr=a.lr, seed=1000 + a.slot, base=self.base)
        if a.load:
            m.load(a.load)
        self.managers[a.name] = m

    def _retire(self, a: AdapterSpec) -> None:
        m = self.managers.pop(a.name, None)
        if m is None:
            return
        if self.save_dir:
            m.save(os.path.join(self.save_dir, a.name, f"final_step_{a.steps}"))
        if self.active == a.name:
            self._restore_base(m)
            self.active = None

    def _base_store(self):
        if self.active is not None:  # base copies are taken from the live weights: they must be the base weights now
            self._restore_base(self.managers[self.active])
            self.active = None
        return self.actor.store

    def _restore_base(self, m: LoRAManager) -> None:
        import torch

        with torch.no_grad():
            for n, b in m.base.items():
                self.actor.store.params[n].copy_(b)
        self.actor.store.version += 1

    # ------------------------------------------------------------------ per-step use
    def activate(self, name: str) -> LoRAManager:
        """Make ``name`` the adapter whose merged weights are live (trainer and colocated engine)."""
        m = self.managers[name]
        if self.active != name:
            m.merge()  # merge() starts from the stored base copies, so it also undoes the previous adapter
            self.actor.store.version += 1
            self.active = name
        self.actor.lora = m
        return m

    def after_train(self, name: str, rollout_id: int, save_interval: Optional[int] = None) -> bool:
        """Counts the step and writes the periodic adapter checkpoint. Returns True when the adapter has reached its
        ``num_step`` (the caller deregisters it)."""
        done = self.registry.bump_steps(name)
        a = self.registry.get(name)
        if self.save_dir and save_interval and a.steps % save_interval == 0:
            self.managers[name].save(os.path.join(self.save_dir, name, f"step_{a.steps}"))
        return done


def build_control_app(registry: AdapterRegistry, on_change: Optional[Callable[[], None]] = None):
    """FastAPI app: ``GET /adapters``, ``POST /adapters`` (JSON AdapterSpec fields), ``DELETE /adapters/{name}``."""
    from fastapi import FastAPI, HTTPException, Request

    app = FastAPI(title="miles_b200 multi-LoRA control")

    @app.get("/adapters")
    async def list_adapters():
        version, specs = registry.snapshot()
        return {"version": version, "adapters": [a.to_dict() for a in specs]}

    @app.post("/adapters")
    async def register(req: Request):
        body = await req.json()
        try:
            spec = registry.register(AdapterSpec(**{k: v for k, v in body.items() if k in AdapterSpec.__dataclass_fields__
                                                    and k not in ("state", "slot", "steps", "registration_id")}))
        except (ValueError, RuntimeError, TypeError) as e:
            raise HTTPException(409, str(e))
        if on_change:
            on_change()
        return spec.to_dict()

    @app.delete("/adapters/{name}")
    async def deregister(name: str):
        try:
            a = registry.deregister(name)
        except KeyError:
            raise HTTPException(404, f"unknown adapter {name}")
        if on_change:
            on_change()
        return a.to_dict()

    return app
