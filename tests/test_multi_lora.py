"""Multi-LoRA registry state machine, controller reconciliation on a tiny CPU model, HTTP control API."""
import pytest
import torch

from miles_b200.models import ParamStore, get_config
from miles_b200.multi_lora import AdapterRegistry, AdapterSpec, AdapterState, MultiLoRAController, build_control_app


class _Actor:
    def __init__(self):
        self.cfg = get_config("qwen3-tiny")
        self.store = ParamStore(self.cfg, "cpu", torch.float32, seed=1)
        self.store.allocate_grads(torch.float32)
        self.lora = None


def test_registry_slots_and_transitions():
    r = AdapterRegistry(max_slots=2)
    a = r.register(AdapterSpec("a"))
    b = r.register(AdapterSpec("b", rank=8))
    assert (a.slot, b.slot) == (0, 1)
    with pytest.raises(ValueError):
        r.register(AdapterSpec("a"))
    with pytest.raises(RuntimeError):
        r.register(AdapterSpec("c"))
    r.transition("a", AdapterState.ACTIVE)
    with pytest.raises(ValueError):
        r.transition("a", AdapterState.REMOVED)  # an active adapter must drain first
    assert r.deregister("a").state == AdapterState.DRAINING
    assert r.deregister("b").state == AdapterState.REMOVED  # never activated: removed at once
    r.transition("a", AdapterState.REMOVED)
    assert r.snapshot()[1] == [] and r.register(AdapterSpec("c")).slot == 0


def test_controller_switches_adapters_on_one_base(tmp_path):
    actor = _Actor()
    base = {n: p.clone() for n, p in actor.store.params.items()}
    ctl = MultiLoRAController(actor, AdapterRegistry(4), save_dir=str(tmp_path))
    ctl.registry.register(AdapterSpec("x", rank=4, target_modules=["q_proj", "down_proj"]))
    ctl.registry.register(AdapterSpec("y", rank=2, target_modules=["q_proj"]))
    assert ctl.reconcile() == ["x", "y"]
    mx, my = ctl.managers["x"], ctl.managers["y"]
    assert mx.base is my.base  # one shared copy of the base tensors
    with torch.no_grad():
        for b in mx.B:
            b.normal_(0, 0.1)
        for b in my.B:
            b.normal_(0, 0.1)
    ctl.activate("x")
    wx = actor.store.params["layers.0.attn.qkv.weight"].clone()
    assert not torch.equal(wx, base["layers.0.attn.qkv.weight"]) and actor.lora is mx
    ctl.activate("y")
    wy = actor.store.params["layers.0.attn.qkv.weight"].clone()
    assert not torch.equal(wy, wx)
    assert torch.equal(actor.store.params["layers.0.mlp.down.weight"], base["layers.0.mlp.down.weight"])  # y does not touch it
    ctl.activate("x")
    assert torch.equal(actor.store.params["layers.0.attn.qkv.weight"], wx)
    ctl.after_train("x", 0, save_interval=1)
    assert (tmp_path / "x" / "step_1" / "adapter_model.safetensors").exists()
    ctl.registry.deregister("x")
    assert ctl.reconcile() == ["y"] and "x" not in ctl.managers
    assert torch.equal(actor.store.params["layers.0.attn.qkv.weight"], base["layers.0.attn.qkv.weight"])  # base restored


def test_http_control_api():
    from fastapi.testclient import TestClient

    reg = AdapterRegistry(2)
    c = TestClient(build_control_app(reg))
    assert c.post("/adapters", json={"name": "m", "rank": 8, "lr": 2e-4}).json()["slot"] == 0
    assert c.post("/adapters", json={"name": "m"}).status_code == 409
    assert [a["name"] for a in c.get("/adapters").json()["adapters"]] == ["m"]
    assert c.delete("/adapters/m").json()["state"] == "removed"
    assert c.delete("/adapters/nope").status_code == 404
