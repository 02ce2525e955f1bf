"""Dashboard store partitions, collector sinks, advisory rules, HTTP endpoints."""
import time

from miles_b200.dashboard import Collector, EventStore, advisories, build_dashboard_app


def test_store_partitions_and_torn_lines(tmp_path):
    s = EventStore(str(tmp_path))
    t0 = time.time()
    s.append("metrics", {"step": 0}, t=t0 - 7200)
    s.append("metrics", {"step": 1}, t=t0 - 10)
    s.append("metrics", {"step": 2}, t=t0)
    parts = sorted((tmp_path / "metrics").iterdir())
    assert len(parts) >= 2  # two hours apart: different partitions
    with open(parts[-1], "a") as f:
        f.write('{"t": 1, "step"')  # torn line from a crash
    assert [r["step"] for r in s.read("metrics", since=t0 - 100)] == [1, 2]
    assert [r["step"] for r in s.tail("metrics", 2)] == [1, 2] and s.streams() == ["metrics"]


def test_collector_and_advisories_and_http(tmp_path):
    from fastapi.testclient import TestClient

    s = EventStore(str(tmp_path))
    c = Collector(s, gpu_sampler=lambda: [{"gpu": 0, "util": 99, "mem_used": 1, "mem_total": 2, "power_w": 900.0, "sm_mhz": 600}])
    for i in range(6):
        c.log_metrics({"perf/rollout_time": 60.0, "perf/train_time": 10.0, "train/grad_norm": 1.0 if i < 5 else 50.0,
                       "train/train_rollout_logprob_abs_diff": 0.2, "note": "text is dropped"}, step=i)
    c.on_lifecycle({"event": "attempt_end", "sample_index": 3, "t": time.time()})
    assert c.sample_gpus_once() == 1
    rules = {a["rule"] for a in advisories(s)}
    assert {"rollout_bound", "train_rollout_mismatch", "grad_spike", "low_clocks"} <= rules
    app = TestClient(build_dashboard_app(s))
    assert "miles_b200" in app.get("/").text
    assert set(app.get("/api/streams").json()) == {"gpus", "metrics", "trajectories"}
    assert len(app.get("/api/metrics?limit=3").json()) == 3
    assert any(a["rule"] == "grad_spike" for a in app.get("/api/advisories").json())


def test_engine_scrape_and_advisories(tmp_path):
    from miles_b200.dashboard.collector import Collector, advisories, parse_prometheus
    from miles_b200.dashboard.store import EventStore

    text = '# HELP x\nmiles_b200:num_running_reqs 2\nmiles_b200:num_queue_reqs{engine="0"} 40\nbad line\n'
    assert parse_prometheus(text) == {"miles_b200:num_running_reqs": 2.0, "miles_b200:num_queue_reqs": 40.0}
    st = EventStore(str(tmp_path))
    col = Collector(st, gpu_sampler=lambda: [])
    col.add_engine("http://e0/")
    col.add_engine("http://e1")

    def fetch(url):
        if "e1" in url:
            raise OSError("refused")
        return text

    assert col.scrape_engines_once(fetch) == 1
    rules = {a["rule"] for a in advisories(st)}
    assert {"engine_down", "engine_queue"} <= rules


def test_timeline_and_rollout_inspector_endpoints(tmp_path):
    import os

    import torch
    from fastapi.testclient import TestClient

    from miles_b200.dashboard.serve import build
    from miles_b200.utils.types import Sample

    root = str(tmp_path)
    s = EventStore(os.path.join(root, "dashboard"))
    c = Collector(s, gpu_sampler=lambda: [{"gpu": g, "util": 50 + g, "mem_used": 1, "mem_total": 2, "power_w": 500.0, "sm_mhz": 1900} for g in (0, 1)])
    for i in range(3):
        c.log_metrics({"perf/rollout_time": 6.0, "perf/train_time": 3.0, "perf/train_fwd_bwd_time": 2.0, "perf/update_weights_time": 0.1,
                       "perf/step_time": 10.0, "perf/train_wait_time": 0.5}, step=i)
    c.sample_gpus_once()
    os.makedirs(os.path.join(root, "rollout_data"))
    samples = []
    for g in range(2):
        for k in range(3):
            sm = Sample(index=g * 3 + k, group_index=g, prompt="what is 2+2?", tokens=[5, 6, 7, 10 + k, 11 + k], response="four", response_length=2,
                        reward=float(k % 2) if g == 0 else 1.0, rollout_log_probs=[-0.5, -0.25], loss_mask=[1, 0], weight_versions=[3])
            sm.status = Sample.Status.COMPLETED
            samples.append(sm.to_dict())
    torch.save({"rollout_id": 0, "samples": samples}, os.path.join(root, "rollout_data", "0.pt"))
    app = TestClient(build(root))
    meta = app.get("/api/meta").json()
    assert meta["rollout_dumps"] == [0] and meta["last_step"] == 2 and "metrics" in meta["streams"]
    ph = app.get("/api/timeline/phases").json()
    assert len(ph) == 3 and ph[0]["rollout_time"] == 6.0 and ph[0]["train_fwd_bwd_time"] == 2.0
    bub = app.get("/api/timeline/bubbles").json()
    assert abs(bub[0]["unaccounted_s"] - 0.9) < 1e-9 and abs(bub[0]["wait_ratio"] - 0.05) < 1e-9
    assert set(app.get("/api/timeline/gpu").json()) == {"0", "1"}
    summ = app.get("/api/rollout/0/summary").json()
    assert summ["num_samples"] == 6 and summ["num_groups"] == 2 and summ["weight_versions"] == [3] and summ["response_len_max"] == 2
    groups = app.get("/api/rollout/0/groups").json()
    assert [g["all_equal"] for g in groups] == [False, True] and groups[0]["rewards"] == [0.0, 1.0, 0.0]
    toks = app.get("/api/rollout/0/sample/4/tokens").json()
    assert toks["prompt_tokens"] == 3 and [t["id"] for t in toks["tokens"]] == [11, 12] and toks["tokens"][1]["loss_mask"] == 0
    msgs = app.get("/api/rollout/0/sample/1/messages").json()["messages"]
    assert msgs[0]["role"] == "user" and msgs[-1] == {"role": "assistant", "content": "four"}
    assert app.get("/api/rollout/7/summary").status_code == 404 and app.get("/api/rollout/0/sample/99/tokens").status_code == 404


def test_dashboard_flags_configure_the_collector(tmp_path):
    """--use-miles-dashboard and the --dashboard-* flags of the reference: header snapshot, sampling cadences, engine metric
    whitelist, forwarding of the collector's gauges."""
    import json

    import pytest

    from miles_b200.utils.arguments import parse_args
    from miles_b200.utils.tracking import DashboardBackend, init_tracking

    base = ["--model-preset", "qwen3-tiny", "--num-rollout", "1", "--rollout-batch-size", "2", "--n-samples-per-prompt", "2"]
    with pytest.raises(ValueError):
        init_tracking(parse_args(base + ["--use-miles-dashboard"]), primary=True)
    a = parse_args(base + ["--use-miles-dashboard", "--dump-details", str(tmp_path), "--dashboard-gpu-sample-interval", "0.5",
                           "--dashboard-sglang-scrape-interval", "0.25", "--dashboard-sglang-metrics", "num_running_reqs,gen_throughput",
                           "--rollout-engine-urls", "http://127.0.0.1:1"])
    seen = []
    b = DashboardBackend(str(tmp_path / "dashboard"), a, forward=lambda n, v, l: seen.append((n, v, l)))
    try:
        c = b.collector
        assert (c.gpu_interval, c.engine_interval, c.engine_metrics) == (0.5, 0.25, {"num_running_reqs", "gen_throughput"})
        meta = json.load(open(tmp_path / "dashboard" / "meta.json"))
        assert meta["model_preset"] == "qwen3-tiny" and meta["rollout_batch_size"] == 2
        n = c.scrape_engines_once(fetch=lambda url: "num_running_reqs 3\nother_metric 9\ngen_throughput{engine=\"0\"} 120.5\n")
        assert n == 1
        rows = list(c.store.read("engines"))
        assert rows[-1]["num_running_reqs"] == 3.0 and rows[-1]["gen_throughput"] == 120.5 and "other_metric" not in rows[-1]
        assert ("dashboard_engine_gen_throughput", 120.5, {"engine": "http://127.0.0.1:1"}) in seen
    finally:
        b.finish()
