"""Host-side fault tolerance (cells, health checks, controller), router policies, async data buffer, rewards."""
import asyncio

import pytest

from miles_b200.ft.cells import CellState, StepResult, TrainGroup
from miles_b200.ft.control_server import MiniFTController
from miles_b200.ft.fault_injector import InjectedFault, inject, parse_actions
from miles_b200.ft.health import HealthMonitor, SimpleHealthChecker, SimpleHeartbeat
from miles_b200.rollout.fully_async_rollout import DefaultDataBuffer
from miles_b200.rollout.rm_hub import async_rm
from miles_b200.router.router import MilesRouter
from miles_b200.utils.types import Sample


class DummyActor:
    """Records every call; fails on demand (host-side exception only)."""

    def __init__(self, cell: int, log: list, fail_plan: dict):
        self.cell, self.log, self.fail_plan = cell, log, fail_plan
        self.state = {"w": 0}
        self.killed = False

    def init(self, quorum_id):
        self.log.append(("init", self.cell, quorum_id))

    def reconfigure(self, quorum_id, members):
        self.log.append(("reconfigure", self.cell, quorum_id, tuple(members)))

    def send_ckpt(self):
        return dict(self.state)

    def recv_ckpt(self, ckpt):
        self.state = dict(ckpt)
        self.log.append(("recv_ckpt", self.cell, ckpt["w"]))

    def train(self, rollout_id, data, attempt=0):
        key = (self.cell, rollout_id)
        if self.fail_plan.get(key, 0) > 0:
            self.fail_plan[key] -= 1
            raise InjectedFault(f"cell {self.cell} crashed before all-reduce")
        self.state["w"] += 1
        self.log.append(("train", self.cell, rollout_id, attempt, data))
        return StepResult("NORMAL", self.state["w"])

    def discard_step(self, rollout_id):
        self.log.append(("discard", self.cell, rollout_id))

    def kill(self):
        self.killed = True


def test_cells_retry_heal_and_checkpoint_transfer():
    log, fail = [], {(1, 1): 1}
    group = TrainGroup(2, lambda i: [DummyActor(i, log, fail)], max_retries=5)
    group.init()
    assert [c.state for c in group.cells] == [CellState.ALLOCATED_ALIVE] * 2 and group.quorum_id == 1
    group.train_step(0, lambda rank, n: (rank, n))
    # step 1: cell 1 crashes -> step discarded on the survivor, cell healed from the survivor's checkpoint, retried
    res = group.train_step(1, lambda rank, n: (rank, n))
    assert len(res) == 2 and group.quorum_id == 2
    assert ("discard", 0, 1) in log
    assert any(e[0] == "recv_ckpt" and e[1] == 1 for e in log)
    assert ("healed", 1, 2) in group.events
    trains = [e for e in log if e[0] == "train" and e[2] == 1]
    assert {e[1] for e in trains} == {0, 1} and max(e[3] for e in trains) == 1
    # suspend / resume through the controller
    group.suspend(0)
    assert group.cells[0].state == CellState.STOPPED
    res = group.train_step(2, lambda rank, n: (rank, n))
    assert len(res) == 1
    group.resume(0)
    group.refresh_cells()
    assert group.cells[0].alive and len(group.train_step(3, lambda r, n: (r, n))) == 2


def test_health_checker_heartbeat_monitor_and_controller():
    t = [0.0]
    hb = SimpleHeartbeat(clock=lambda: t[0])
    hb.bump("train")
    t[0] = 12.0
    assert hb.age() == 12.0 and hb.status()["phase"] == "train"
    seq = iter([True, False, False, True, False, False, False, True])
    events = []
    hc = SimpleHealthChecker(lambda: next(seq), lambda: events.append("down"), lambda: events.append("up"), failure_threshold=3)
    states = [hc.check_once() for _ in range(8)]
    assert states == [True, True, True, True, True, True, False, True] and events == ["down", "up"]

    class Eng:
        def __init__(self, ok):
            self.ok = ok

        def health_generate(self):
            if self.ok == "raise":
                raise RuntimeError("connection refused")
            return self.ok

    killed = []
    mon = HealthMonitor([Eng(True), Eng(False), Eng("raise")], killed.append, timeout=1.0)
    assert mon.check_all() == [1, 2] and killed == [1, 2] and mon.check_all() == []
    mon.mark_recovered(1, Eng(True))
    assert mon.check_all() == []

    log = []
    group = TrainGroup(2, lambda i: [DummyActor(i, log, {})])
    group.init()
    healthy = {0: True, 1: False}
    ctl = MiniFTController(group, lambda i: healthy[i], resume_delay=10.0, clock=lambda: t[0])
    ctl.poll_once()
    assert group.cells[1].suspended
    healthy[1] = True
    t[0] += 5
    ctl.poll_once()
    assert group.cells[1].suspended
    t[0] += 6
    ctl.poll_once()
    assert not group.cells[1].suspended


def test_fault_injector_host_side_only():
    with pytest.raises(InjectedFault):
        inject("exception")
    with pytest.raises(ValueError):
        inject("gpu_trap")
    acts = parse_actions("stop_cell_at_end:1:3,crash_before_allreduce:0:2")
    assert [(a.kind, a.cell, a.rollout_id) for a in acts] == [("stop_cell_at_end", 1, 3), ("crash_before_allreduce", 0, 2)]


def test_router_policies_and_quarantine():
    r = MilesRouter(failure_threshold=2)
    for u in ("http://a", "http://b", "http://c"):
        r.add_worker(u)
    for _ in range(9):  # least-inflight spreads them 3 / 3 / 3; finishing some leaves a = 3, b = 1, c = 2
        r.acquire()
    for u, n in (("http://b", 2), ("http://c", 1)):
        for _ in range(n):
            r.release(u, True)
    assert r.workers == {"http://a": 3, "http://b": 1, "http://c": 2}
    assert r.pick() == "http://b"
    r.mark_result("http://b", False)
    assert r.pick() == "http://b"
    r.mark_result("http://b", False)
    assert "http://b" in r.dead and r.pick() == "http://c"
    r.policy = "consistent_hashing"
    assert r.pick("session-1") == r.pick("session-1")
    r.policy = "round_robin"
    assert {r.pick() for _ in range(4)} == {"http://a", "http://c"}
    r.remove_worker("http://a")
    r.remove_worker("http://c")
    with pytest.raises(RuntimeError):
        r.pick()


class _Args:
    rollout_batch_size = 2
    n_samples_per_prompt = 2
    async_data_buffer_capacity_factor = 2
    max_weight_staleness = 1
    async_unused_samples_handler = "retry"
    rm_type = "deepscaler"
    custom_rm_path = None
    reward_key = None


class _DS:
    def __init__(self):
        self.added = []

    def add_samples(self, groups):
        self.added += groups


def _group(idx, version, status=Sample.Status.COMPLETED):
    return [Sample(group_index=idx, index=2 * idx + j, tokens=[1, 2, 3, 4], response_length=2, reward=1.0,
                   weight_versions=[version], status=status) for j in range(2)]


def test_async_buffer_filters_and_staleness():
    ds = _DS()
    buf = DefaultDataBuffer(_Args(), ds)
    assert buf.capacity == 4
    assert not buf.put(_group(0, 5, Sample.Status.ABORTED))
    for i, v in enumerate((3, 5, 6)):
        assert buf.put(_group(i + 1, v))
    got = buf.get(2, current_version=6)
    assert [g[0].group_index for g in got] == [2, 3]  # version 3 lags by 3 > 1: recycled to the data source
    assert buf.stats["retried_stale"] == 1 and len(ds.added) == 1
    fresh = ds.added[0][0]
    assert fresh.response_length == 0 and fresh.tokens == [1, 2] and fresh.reward is None and fresh.weight_versions == []


def test_math_and_misc_rewards():
    a = _Args()
    s = Sample(response="<think>hmm</think> so the answer is \\boxed{\\frac{3}{4}}", label="0.75")
    assert asyncio.run(async_rm(a, s)) == 1.0
    s = Sample(response="\\boxed{7}", label="8")
    assert asyncio.run(async_rm(a, s)) == 0.0
    a.rm_type = "dapo"
    assert asyncio.run(async_rm(a, s)) == -1.0
    a.rm_type = "parity"
    assert asyncio.run(async_rm(a, Sample(tokens=[9, 1, 3], response_length=2))) == 1.0
    a.rm_type = "f1"
    assert asyncio.run(async_rm(a, Sample(response="the cat sat", label="cat sat down"))) == pytest.approx(0.8)
    a.rm_type = "deterministic_random"
    s = Sample(prompt="p", response="r")
    assert asyncio.run(async_rm(a, s)) == asyncio.run(async_rm(a, s))


def test_control_server_and_router_over_http():
    """The JSON-body endpoints answer through a real HTTP stack (request objects are resolved by the framework)."""
    from fastapi.testclient import TestClient

    from miles_b200.ft.cells import TrainGroup
    from miles_b200.ft.control_server import build_control_app
    from miles_b200.router.router import MilesRouter, build_router_app

    class Actor:
        def __init__(self):
            self.faults = []

        def init(self):
            return 0

        def inject_fault(self, kind):
            self.faults.append(kind)

    actors = {}

    def factory(i):
        actors[i] = Actor()
        return [actors[i]]

    group = TrainGroup(2, factory)
    group.init()
    c = TestClient(build_control_app(group))
    cells = c.get("/api/v1/cells").json()
    name = (cells["items"] if isinstance(cells, dict) else cells)[0]["metadata"]["name"]
    r = c.patch(f"/api/v1/cells/{name}", json={"spec": {"suspend": True}})
    assert r.status_code == 200
    r = c.post(f"/api/v1/cells/{name}/inject-fault", json={"type": "exception"})
    assert r.status_code == 200 and "delivered" in r.json()
    assert c.post(f"/api/v1/cells/{name}/inject-fault", json={"type": "segfault"}).status_code == 400  # host-side faults only

    router = MilesRouter(health_interval=3600)

    async def fake_forward(method, path, body, headers):
        return 200, b'{"echo": "' + path.encode() + b'"}', "application/json"

    router.forward = fake_forward
    rc = TestClient(build_router_app(router))
    assert rc.post("/add_worker", params={"url": "http://w0"}).status_code == 200
    r = rc.post("/generate", json={"input_ids": [1, 2]})
    assert r.status_code == 200 and r.json() == {"echo": "/generate"}


def test_fault_tolerance_runtime_in_the_loop(tmp_path):
    """--use-fault-tolerance: training goes through the cell group; a scripted crash before the gradient reduction is
    retried, a scripted stop drops a rollout's training and a scripted start brings the cell back; the control server
    lists the cell."""
    import json
    import socket
    import urllib.request

    from miles_b200.loop import RLLoop
    from miles_b200.utils.arguments import parse_args

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    actions = [{"at_rollout": 0, "action": "crash_before_allreduce", "cell_index": 0},
               {"at_rollout": 1, "action": "stop_cell_at_end", "cell_index": -1},
               {"at_rollout": 2, "action": "start_cell_at_end", "cell_index": 0}]
    args = parse_args(["--model-preset", "qwen3-tiny", "--num-rollout", "4", "--rollout-batch-size", "2", "--n-samples-per-prompt", "2",
                       "--rollout-max-response-len", "8", "--rm-type", "parity", "--advantage-estimator", "grpo", "--lr", "1e-4",
                       "--colocate", "--actor-num-gpus-per-node", "1", "--use-fault-tolerance", "--control-server-port", str(port),
                       "--mini-ft-controller-enable", "--ci-ft-test-actions", json.dumps(actions)])
    loop = RLLoop(args)
    cells = json.loads(urllib.request.urlopen(f"http://127.0.0.1:{port}/api/v1/cells", timeout=5).read())
    assert [c["metadata"]["name"] for c in cells["items"]] == ["cell-0"]
    hist = loop.run()
    assert len(hist) == 4
    events = loop.ft.group.events
    assert any(e[0] == "cell_error" for e in events), events        # rollout 0: the injected crash was seen ...
    assert ("step_ok", 0, 1) in events                              # ... and the step succeeded on the retry
    assert "train/grad_norm" in hist[0] and "train/grad_norm" in hist[1]
    assert hist[2].get("train/skipped_suspended") == 1.0            # stopped at the end of rollout 1
    assert "train/grad_norm" in hist[3]                             # started again at the end of rollout 2
