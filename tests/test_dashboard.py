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
