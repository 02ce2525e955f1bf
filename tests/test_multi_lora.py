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


def test_service_trains_each_adapter_on_its_own_data_batch_and_lifetime(tmp_path):
    """Two adapters on one base model: different prompt files, batch sizes and reward types; one retires after its
    num_step (derived from num_epoch for the other), both are saved, and the base weights are back afterwards."""
    import json

    from miles_b200.loop import RLLoop
    from miles_b200.multi_lora import AdapterDataSources, run_service, train_adapter_step
    from miles_b200.utils.arguments import parse_args

    def prompts(path, first_token, n):
        with open(path, "w") as f:
            for i in range(n):
                f.write(json.dumps({"input": [first_token, 10 + i, 11 + i, 12 + i], "label": "1"}) + "\n")

    prompts(tmp_path / "a.jsonl", 100, 8)
    prompts(tmp_path / "b.jsonl", 200, 4)
    args = parse_args(["--model-preset", "qwen3-tiny", "--rollout-batch-size", "4", "--n-samples-per-prompt", "2", "--rollout-max-response-len", "6",
                       "--rollout-max-prompt-len", "16", "--rm-type", "parity", "--lr", "1e-4", "--micro-batch-size", "8", "--colocate",
                       "--num-rollout", "10", "--actor-num-gpus-per-node", "1", "--save", str(tmp_path / "out"), "--input-key", "input",
                       "--label-key", "label"])
    loop = RLLoop(args)
    base = {n: p.clone() for n, p in loop.actor.store.params.items()}
    reg = AdapterRegistry(max_slots=4, samples_per_prompt=2)
    ctl = MultiLoRAController(loop.actor, reg, save_dir=str(tmp_path / "out"))
    reg.register(AdapterSpec("a", rank=4, prompt_data=str(tmp_path / "a.jsonl"), rollout_batch_size=4, rm_type="random", num_step=3))
    reg.register(AdapterSpec("b", rank=2, prompt_data=str(tmp_path / "b.jsonl"), rollout_batch_size=2, num_epoch=1.0))
    sources = AdapterDataSources(args, loop.tokenizer, lambda a, tok: loop._build_data_source_for(a), reg, default_batch=args.rollout_batch_size)
    assert ctl.reconcile() == ["a", "b"]
    sources.reconcile(reg.snapshot()[1])
    assert reg.get("b").num_step == 2 and reg.get("a").registration_id != reg.get("b").registration_id   # 4 prompts / 2 per step
    seen = {"a": [], "b": []}
    orig_train = loop.train

    def spy(rid, samples):
        seen[samples[0].metadata["adapter"]].append(samples)
        return orig_train(rid, samples)

    loop.train = spy
    logs = []
    n = run_service(loop, ctl, sources, max_rollouts=10, can_register=False, log=logs.append)
    assert n == 5 and [len(v) for v in seen.values()] == [3, 2]              # a: 3 steps, b: 2 steps, then nobody is left
    assert all(len(s) == 8 for s in seen["a"]) and all(len(s) == 4 for s in seen["b"])   # 4 x 2 and 2 x 2 samples per step
    assert all(s.tokens[0] == 100 and s.metadata["rm_type"] == "random" for step in seen["a"] for s in step)
    assert all(s.tokens[0] == 200 and "rm_type" not in s.metadata for step in seen["b"] for s in step)
    assert reg.snapshot()[1] == [] and not ctl.managers
    assert (tmp_path / "out" / "a" / "final_step_3" / "adapter_model.safetensors").exists()
    assert (tmp_path / "out" / "b" / "final_step_2" / "adapter_model.safetensors").exists()
    assert any("(retired)" in l for l in logs)
    for name, p in loop.actor.store.params.items():
        assert torch.allclose(p, base[name], atol=1e-6), name                # the base model never moved
    assert loop.actor.args.global_batch_size == args.global_batch_size and loop.rollout_fn.args.rollout_batch_size == 4
