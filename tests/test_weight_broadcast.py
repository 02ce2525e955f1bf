"""Weight update over a dedicated process group (gloo, two processes) and the engine endpoints around it."""
import socket

import torch
import torch.multiprocessing as mp

from miles_b200.models import ParamStore, get_config
from miles_b200.weight_sync.broadcast import (bucket_header, destroy_update_group, init_update_group, iter_buckets,
                                              receive_bucket, send_bucket)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_iter_buckets_respects_the_byte_limit():
    ts = [(f"t{i}", torch.zeros(n)) for i, n in enumerate([10, 10, 100, 5, 5, 5])]
    bs = list(iter_buckets(ts, 100))  # 100 bytes = 25 floats
    assert [[n for n, _ in b] for b in bs] == [["t0", "t1"], ["t2"], ["t3", "t4", "t5"]]


def _proc(rank, port, q_hdr, ret):
    torch.set_num_threads(2)  # several ranks share the host cores
    cfg = get_config("qwen3-tiny")
    init_update_group("127.0.0.1", port, rank, 2, "w", backend="gloo", timeout_s=60)
    if rank == 0:  # trainer
        src = ParamStore(cfg, "cpu", torch.float32, seed=1)
        for bucket in iter_buckets(src.params.items(), 1 << 20):
            q_hdr.put(bucket_header(bucket, "w"))
            send_bucket(bucket, "w")
        q_hdr.put(None)
        ret[0] = src.checksum()
    else:          # engine
        dst = ParamStore(cfg, "cpu", torch.float32, seed=2)
        n = 0
        while True:
            hdr = q_hdr.get()
            if hdr is None:
                break
            n += receive_bucket(hdr, dst)
        ret[1] = (dst.checksum(), n, len(dst.params))
    assert destroy_update_group("w")


def test_broadcast_update_between_two_processes():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ret = ctx.Manager().dict()
    port = _free_port()
    ps = [ctx.Process(target=_proc, args=(r, port, q, ret)) for r in range(2)]
    for p in ps:
        p.start()
    for p in ps:
        p.join(120)
        assert p.exitcode == 0
    (chk, n, total) = ret[1]
    assert n == total and chk == ret[0]


def test_engine_endpoints_adapters_profile_and_layout(tmp_path):
    from fastapi.testclient import TestClient

    from miles_b200.engine import Engine
    from miles_b200.engine.server import build_app
    from miles_b200.lora import LoRAManager
    from miles_b200.models import build_model
    from miles_b200.weight_sync.disk_delta import DiskDeltaWriter
    from miles_b200.weight_sync.registry import put_bucket

    cfg = get_config("qwen3-tiny")
    st = ParamStore(cfg, "cpu", torch.float32, seed=11)
    eng = Engine(build_model(cfg, st), max_running=2, page_size=8, max_seq_len=64)
    c = TestClient(build_app(eng))
    assert c.get("/parallelism_config").json()["tp_size"] == 1
    # adapter round trip: load changes the weights, unload restores them
    other = ParamStore(cfg, "cpu", torch.float32, seed=11)
    lm = LoRAManager(other, 4, 8, "all-linear", lr=1e-3, weight_decay=0.0, seed=3)
    for b in lm.B:
        b.data.normal_(0, 0.05)
    before = {g: t.clone() for g, t in st.flat.items()}
    bid = put_bucket(lm.adapter_tensors())
    r = c.post("/load_lora_adapter_from_tensors", json={"lora_name": "a1", "bucket_id": bid, "scaling": lm.scale})
    assert r.status_code == 200 and r.json()["loaded_adapters"] == ["a1"]
    assert not torch.equal(st.flat["dense"], before["dense"])
    lm.merge()
    assert torch.allclose(st.flat["dense"], other.flat["dense"], atol=1e-5)  # same result as the trainer-side merge
    assert c.post("/unload_lora_adapter", json={"lora_name": "a1"}).status_code == 200
    assert torch.allclose(st.flat["dense"], before["dense"], atol=1e-5)
    assert c.post("/unload_lora_adapter", json={"lora_name": "a1"}).status_code == 404
    # profile
    assert c.post("/start_profile", json={"output_dir": str(tmp_path), "activities": ["CPU"]}).status_code == 200
    assert c.post("/start_profile", json={}).status_code == 409
    tr = c.post("/stop_profile").json()["trace"]
    import os

    assert os.path.exists(tr)
    # pull a published delta
    new = ParamStore(cfg, "cpu", torch.float32, seed=99)
    w = DiskDeltaWriter(str(tmp_path / "delta"), encoding="overwrite")
    w.write(list(new.params.items()), version=1)
    r = c.post("/pull_weights", json={"path": str(tmp_path / "delta" / "v00000001"), "weight_version": 1})
    assert r.status_code == 200 and r.json()["num_tensors"] == len(new.params)
    assert torch.equal(st.flat["dense"], new.flat["dense"]) and eng.weight_version == 1


def _serve(port, ready):
    torch.set_num_threads(2)
    from miles_b200.engine import Engine
    from miles_b200.engine.server import serve
    from miles_b200.models import build_model

    cfg = get_config("qwen3-tiny")
    st = ParamStore(cfg, "cpu", torch.float32, seed=2)  # starts from other weights than the trainer
    eng = Engine(build_model(cfg, st), max_running=2, page_size=8, max_seq_len=64)
    ready.set()
    serve(eng, port=port)


def test_updater_drives_an_engine_server_in_another_process():
    """The whole disaggregated path: HTTP announcements + broadcasts on a dedicated gloo group."""
    import time
    from types import SimpleNamespace as NS

    from miles_b200.weight_sync.broadcast import BroadcastWeightUpdater, HttpEngineHandle

    ctx = mp.get_context("spawn")
    port = _free_port()
    ready = ctx.Event()
    srv = ctx.Process(target=_serve, args=(port, ready), daemon=True)
    srv.start()
    try:
        assert ready.wait(120)
        h = HttpEngineHandle(f"http://127.0.0.1:{port}", timeout_s=60)
        for _ in range(100):  # the HTTP server comes up a moment after the engine is built
            try:
                h.get("/health")
                break
            except Exception:
                time.sleep(0.2)
        cfg = get_config("qwen3-tiny")
        src = ParamStore(cfg, "cpu", torch.float32, seed=1)
        src.version = 4
        actor = NS(store=src, on_gpu=False, args=NS(pause_generation_mode="retract"), ps=None)
        before = h.post("/weights_checker", {"action": "checksum"})["checksum"]
        up = BroadcastWeightUpdater(actor, [h], group_name="w-http", buffer_bytes=1 << 20, backend="gloo")
        m = up.update()
        after = h.post("/weights_checker", {"action": "checksum"})["checksum"]
        want = src.checksum()
        assert before != after and all(abs(after[g] - want[g]) <= 1e-3 * max(1.0, abs(want[g])) for g in want)
        assert h.get("/get_weight_version")["weight_version"] == 4 and m["perf/update_weights_bytes"] > 0
        # a second update reuses the group
        src.flat["dense"].add_(0.25)
        src.version = 5
        up.update()
        after2 = h.post("/weights_checker", {"action": "checksum"})["checksum"]
        assert abs(after2["dense"] - src.checksum()["dense"]) <= 1e-3 * abs(src.checksum()["dense"])
        up.disconnect()
        # the generation endpoints answer over the same HTTP surface, with the weights that just arrived
        assert h.get("/health_generate")["status"] == "ok"
        out = h.post("/generate", {"input_ids": [1, 2, 3, 4], "sampling_params": {"max_new_tokens": 5, "temperature": 0.0},
                                   "return_logprob": True})
        assert len(out["output_ids"]) == 5 and len(out["meta_info"]["output_token_logprobs"]) == 5
        assert out["meta_info"]["weight_version"] == 5 and out["meta_info"]["finish_reason"]["type"] == "length"
        assert h.post("/pause_generation", {"mode": "abort"})["success"] and h.post("/continue_generation", {})["success"]
        info = h.get("/server_info")
        assert info["stats"]["decode_tokens"] >= 4 and info["stats"]["prefill_tokens"] >= 4  # the first token comes out of the prefill
        h.close()
    finally:
        srv.terminate()
        srv.join(10)


def test_disaggregated_loop_generates_remotely_and_broadcasts_weights():
    """`--rollout-engine-urls`: the trainer process has no engine; it generates over HTTP and pushes weights through
    the dedicated group. On-policy parity (trainer vs rollout log-probs) proves the engine got the right weights."""
    import time

    from miles_b200.loop import RLLoop
    from miles_b200.utils.arguments import parse_args
    from miles_b200.weight_sync.broadcast import HttpEngineHandle

    ctx = mp.get_context("spawn")
    port = _free_port()
    ready = ctx.Event()
    srv = ctx.Process(target=_serve, args=(port, ready), daemon=True)
    srv.start()
    try:
        assert ready.wait(120)
        h = HttpEngineHandle(f"http://127.0.0.1:{port}", timeout_s=60)
        for _ in range(100):
            try:
                h.get("/health")
                break
            except Exception:
                time.sleep(0.2)
        args = parse_args(["--model-preset", "qwen3-tiny", "--num-rollout", "2", "--rollout-batch-size", "4", "--n-samples-per-prompt", "2",
                           "--rollout-max-response-len", "8", "--rollout-max-prompt-len", "16", "--rm-type", "parity", "--lr", "1e-3",
                           "--actor-num-nodes", "1", "--actor-num-gpus-per-node", "1", "--rollout-engine-urls", f"http://127.0.0.1:{port}",
                           "--micro-batch-size", "4"])
        loop = RLLoop(args)
        assert loop.engine is None and loop.weight_updater is not None
        hist = loop.run()
        assert len(hist) == 2 and all(m["train/train_rollout_logprob_abs_diff"] < 1e-5 for m in hist)
        assert h.get("/get_weight_version")["weight_version"] == loop.actor.store.version
        want = loop.actor.store.checksum()
        got = h.post("/weights_checker", {"action": "checksum"})["checksum"]
        assert all(abs(got[g] - want[g]) <= 1e-3 * max(1.0, abs(want[g])) for g in want)
        loop.weight_updater.disconnect()
    finally:
        srv.terminate()
        srv.join(10)


def test_engine_server_cli_starts_and_answers():
    import subprocess
    import sys
    import time

    from miles_b200.weight_sync.broadcast import HttpEngineHandle

    port = _free_port()
    p = subprocess.Popen([sys.executable, "-m", "miles_b200.engine.server", "--model-preset", "qwen3-tiny", "--device", "cpu", "--port", str(port),
                          "--max-running-requests", "2", "--page-size", "8", "--context-length", "64"],
                         env=dict(__import__("os").environ, OMP_NUM_THREADS="2"))
    try:
        h = HttpEngineHandle(f"http://127.0.0.1:{port}", timeout_s=30)
        ok = False
        for _ in range(300):
            try:
                ok = h.get("/health")["status"] == "ok"
                break
            except Exception:
                assert p.poll() is None, "the server process exited"
                time.sleep(0.2)
        assert ok
        out = h.post("/generate", {"input_ids": [5, 6, 7], "sampling_params": {"max_new_tokens": 3, "temperature": 0.0}})
        assert len(out["output_ids"]) == 3
        assert h.get("/parallelism_config")["tp_size"] == 1
    finally:
        p.terminate()
        p.wait(10)


def test_fleet_brings_up_a_deployment_and_restarts_an_engine():
    import asyncio
    from types import SimpleNamespace as NS

    from miles_b200.engine.deployment import Deployment
    from miles_b200.engine.fleet import Fleet
    from miles_b200.engine.remote import RemoteEngineClient

    dep = Deployment.from_dict({"sglang": [
        {"name": "actor", "overrides": {"max_running_requests": 2, "page_size": 8, "context_length": 64},
         "server_groups": [{"worker_type": "regular", "num_gpus": 2, "num_gpus_per_engine": 1}]}]}).resolve(
        NS(hf_checkpoint=None, rollout_num_gpus_per_engine=1))
    fleet = Fleet(dep, model_preset="qwen3-tiny", ports=[_free_port(), _free_port()], device="cpu", env={"OMP_NUM_THREADS": "2"})
    fleet.start(wait_s=120)
    try:
        urls = fleet.urls("actor")
        assert len(urls) == 2 and fleet.updatable_urls() == urls
        client = RemoteEngineClient(urls, max_retries=1)

        async def run():
            outs = await asyncio.gather(*[client.generate({"input_ids": [1, 2, 3], "sampling_params": {"max_new_tokens": 2, "temperature": 0.0}})
                                          for _ in range(4)])
            return outs, await client.health()

        outs, health = asyncio.run(run())
        assert all(len(o["output_ids"]) == 2 for o in outs) and all(health.values())
        # the same requests through a router process in front of both engines
        rurl = fleet.start_router(_free_port(), "actor")
        via = RemoteEngineClient([rurl], max_retries=1)

        async def routed():
            return await asyncio.gather(*[via.generate({"input_ids": [4, 5], "sampling_params": {"max_new_tokens": 2, "temperature": 0.0}})
                                          for _ in range(4)])

        assert all(len(o["output_ids"]) == 2 for o in asyncio.run(routed()))
        import json
        import urllib.request

        with urllib.request.urlopen(rurl + "/list_workers", timeout=5) as r:
            assert sorted(json.loads(r.read().decode())["urls"]) == sorted(urls)
        pid = fleet.engines[0].proc.pid
        fleet.engines[0].proc.kill()
        fleet.engines[0].proc.wait(10)
        assert not fleet.engines[0].alive()
        fleet.restart(0, wait_s=120)
        assert fleet.engines[0].alive() and fleet.engines[0].proc.pid != pid
        assert all(asyncio.run(RemoteEngineClient(urls, max_retries=1).health()).values())
        # weights go to both engines; then the health monitor finds a dead engine, replaces it, the updater reconnects
        # and the fresh engine receives the current weights like the survivor
        from miles_b200.weight_sync.broadcast import BroadcastWeightUpdater, HttpEngineHandle

        src = ParamStore(get_config("qwen3-tiny"), "cpu", torch.float32, seed=1)
        src.version = 3
        actor = NS(store=src, on_gpu=False, args=NS(pause_generation_mode="retract"), ps=None)
        handles = [HttpEngineHandle(u, timeout_s=60) for u in urls]
        up = BroadcastWeightUpdater(actor, handles, group_name="fleet-w", buffer_bytes=1 << 20, backend="gloo")
        up.update()
        recovered = []

        def on_recovered(i, u):
            recovered.append((i, u))
            up.replace_engine(i, HttpEngineHandle(u, timeout_s=60))

        mon = fleet.monitor(recover=True, on_recovered=on_recovered)
        assert mon.check_all() == []
        fleet.engines[1].proc.kill()
        fleet.engines[1].proc.wait(10)
        assert mon.check_all() == [1] and recovered == [(1, urls[1])]
        assert fleet.engines[1].alive() and mon.check_all() == []
        src.flat["dense"].mul_(1.01)
        src.version = 4
        up.update()
        want = src.checksum()
        for hnd in up.engines:
            got = hnd.post("/weights_checker", {"action": "checksum"})["checksum"]
            assert all(abs(got[g] - want[g]) <= 1e-3 * max(1.0, abs(want[g])) for g in want)
            assert hnd.get("/get_weight_version")["weight_version"] == 4
        up.disconnect()
    finally:
        fleet.stop()


def test_loop_launches_its_own_fleet():
    from miles_b200.loop import RLLoop
    from miles_b200.utils.arguments import parse_args

    args = parse_args(["--model-preset", "qwen3-tiny", "--num-rollout", "1", "--rollout-batch-size", "4", "--n-samples-per-prompt", "2",
                       "--rollout-max-response-len", "8", "--rollout-max-prompt-len", "16", "--rm-type", "parity", "--lr", "1e-3",
                       "--actor-num-nodes", "1", "--actor-num-gpus-per-node", "1", "--micro-batch-size", "4",
                       "--launch-rollout-fleet", "--rollout-fleet-device", "cpu", "--rollout-fleet-base-port", str(_free_port()),
                       "--rollout-num-gpus", "1", "--rollout-num-gpus-per-engine", "1", "--use-miles-router"])
    loop = RLLoop(args)
    try:
        assert loop.fleet is not None and len(loop.fleet.engines) == 1 and loop.engine is None
        assert loop.router_url is not None and loop.client.urls == [loop.router_url]  # requests go through the router
        hist = loop.run()
        assert hist[0]["train/train_rollout_logprob_abs_diff"] < 1e-5
    finally:
        if loop.weight_updater is not None and loop.weight_updater.connected:
            loop.weight_updater.disconnect()
        loop.fleet.stop()


def test_async_loop_overlaps_generation_with_training_on_remote_engines():
    from miles_b200.async_loop import AsyncRLLoop
    from miles_b200.utils.arguments import parse_args

    args = parse_args(["--model-preset", "qwen3-tiny", "--num-rollout", "3", "--rollout-batch-size", "4", "--n-samples-per-prompt", "2",
                       "--rollout-max-response-len", "8", "--rollout-max-prompt-len", "16", "--rm-type", "parity", "--lr", "1e-3",
                       "--actor-num-nodes", "1", "--actor-num-gpus-per-node", "1", "--micro-batch-size", "4",
                       "--launch-rollout-fleet", "--rollout-fleet-device", "cpu", "--rollout-fleet-base-port", str(_free_port()),
                       "--rollout-num-gpus", "1", "--rollout-num-gpus-per-engine", "1", "--use-tis"])
    loop = AsyncRLLoop(args)
    started = []
    orig = loop._start_background_generation
    loop._start_background_generation = lambda rid: (started.append(rid), orig(rid))[1]
    try:
        hist = loop.run()
        assert len(hist) == 3 and started == [1, 2]  # rollouts 1 and 2 were generated while 0 and 1 trained
        # a rollout generated during step i used the weights of before step i: one version behind, never more
        assert all(m["train/train_rollout_logprob_abs_diff"] < 0.5 for m in hist)
        assert hist[0]["train/train_rollout_logprob_abs_diff"] < 1e-5
    finally:
        if loop.weight_updater is not None and loop.weight_updater.connected:
            loop.weight_updater.disconnect()
        loop.fleet.stop()


def test_hf_named_pieces_update_fused_parameters_in_any_order():
    """Weights may arrive under HuggingFace tensor names, in any order and split over buckets anyhow: every piece is
    copied into its view of the fused native parameter (so no group of tensors has to arrive atomically)."""
    import random

    import pytest
    import torch

    from miles_b200.models import ParamStore, get_config
    from miles_b200.models.hf_mapping import hf_names, param_or_hf_view

    for name in ("qwen3-tiny", "qwen3-tiny-moe"):
        cfg = get_config(name)
        src = ParamStore(cfg, "cpu", torch.float32, seed=1)
        dst = ParamStore(cfg, "cpu", torch.float32, seed=2)
        items = list(hf_names(cfg, src))
        random.Random(0).shuffle(items)
        for n, t in items:
            param_or_hf_view(cfg, dst, n).copy_(t)
        assert all(torch.equal(src.params[k], dst.params[k]) for k in src.params)
        assert param_or_hf_view(cfg, dst, "final_norm.weight") is dst.params["final_norm.weight"]
        with pytest.raises(KeyError):
            param_or_hf_view(cfg, dst, "model.layers.0.no_such.weight")


def test_generate_endpoint_scores_when_no_token_is_asked_for():
    """POST /generate with max_new_tokens = 0: the engine scores the input (what a distillation teacher and the prefill
    log-prob recomputation ask for) and the prefix cache and request slots are untouched."""
    import torch
    from fastapi.testclient import TestClient

    from miles_b200.engine import Engine
    from miles_b200.engine.server import build_app
    from miles_b200.models import ParamStore, build_model, get_config

    cfg = get_config("qwen3-tiny")
    m = build_model(cfg, ParamStore(cfg, "cpu", torch.float32, seed=11))
    eng = Engine(m, max_running=2, page_size=8, max_seq_len=64, prefix_cache=True)
    c = TestClient(build_app(eng))
    ids = list(range(3, 20))
    r = c.post("/generate", json={"input_ids": ids, "sampling_params": {"max_new_tokens": 0, "temperature": 0}, "return_logprob": True,
                                  "logprob_start_len": 9, "top_logprobs_num": 2}).json()
    meta = r["meta_info"]
    assert r["output_ids"] == [] and meta["completion_tokens"] == 0 and meta["prompt_tokens"] == 17
    assert [e[1] for e in meta["input_token_logprobs"]] == ids[9:] and all(e[0] < 0 for e in meta["input_token_logprobs"])
    assert len(meta["input_top_logprobs"]) == 8 and len(meta["input_top_logprobs"][0]) == 2
    tok, pos, cu = torch.tensor(ids), torch.arange(17), torch.tensor([0, 17])
    lp, _ = m.forward_logprobs(tok, pos, cu, torch.arange(8, 16), tok[9:], 1.0)
    assert torch.allclose(torch.tensor([e[0] for e in meta["input_token_logprobs"]]), lp, atol=1e-5)
    assert not eng.running and eng.prefix.num_pages == 0 and eng.pool.num_free == eng.num_pages - 1


def test_openai_compatible_endpoints_of_the_engine_server():
    from fastapi.testclient import TestClient

    from miles_b200.engine import Engine
    from miles_b200.engine.server import build_app
    from miles_b200.models import build_model

    class Tok:
        chat_template = None

        def __call__(self, text, add_special_tokens=False):
            return {"input_ids": [ord(c) % 250 + 2 for c in text]}

        def decode(self, ids, skip_special_tokens=True):
            return "".join(chr(97 + int(i) % 26) for i in ids)

    cfg = get_config("qwen3-tiny")
    eng = Engine(build_model(cfg, ParamStore(cfg, "cpu", torch.float32, seed=3)), max_running=4, page_size=8, max_seq_len=128)
    with TestClient(build_app(eng, Tok(), "tiny-model")) as c:
        assert c.get("/v1/models").json()["data"][0]["id"] == "tiny-model"
        r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}], "max_tokens": 6, "temperature": 0.0,
                                                 "logprobs": True, "seed": 1}).json()
        ch = r["choices"][0]
        assert r["object"] == "chat.completion" and ch["message"]["role"] == "assistant" and len(ch["message"]["content"]) == 6
        assert ch["finish_reason"] == "length" and len(ch["logprobs"]["content"]) == 6 and r["usage"]["completion_tokens"] == 6
        two = c.post("/v1/completions", json={"prompt": "abc", "max_tokens": 4, "n": 2, "seed": 5}).json()
        assert [len(x["token_ids"]) for x in two["choices"]] == [4, 4] and two["usage"]["prompt_tokens"] == 3
        ids = c.post("/v1/completions", json={"prompt": [5, 6, 7], "max_tokens": 3, "temperature": 0.0}).json()
        direct = c.post("/generate", json={"input_ids": [5, 6, 7], "sampling_params": {"max_new_tokens": 3, "temperature": 0.0}}).json()
        assert ids["choices"][0]["token_ids"] == direct["output_ids"], "the same engine path as /generate"
        s = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}], "max_tokens": 3, "stream": True})
        assert s.headers["content-type"].startswith("text/event-stream") and s.text.strip().endswith("data: [DONE]")
        assert c.post("/v1/chat/completions", json={"messages": []}).status_code == 400
    with TestClient(build_app(eng, None, "")) as c:
        assert c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "x"}]}).status_code == 400
        assert c.post("/v1/completions", json={"prompt": [1, 2], "max_tokens": 2}).status_code == 200
