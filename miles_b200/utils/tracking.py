"""Metric tracking fan-out.

``init_tracking(args)`` builds a ``TrackingManager`` with any of the backends ``wandb``, ``tensorboard``,
``mlflow``, ``prometheus``, ``ci_history`` (JSONL per run, read by the metric-history gates) and
``dashboard`` (append-only JSONL partitions under ``<dump_details>/dashboard``); ``log(metrics, step)``
fans out to all of them.  Optional packages are imported lazily and a missing package disables only its
backend.  Reference: miles/utils/tracking_utils/base.py:23-194, tracking.py:23-56.
"""
from __future__ import annotations

import json
import os
import time
from typing import Optional


class TrackingBackend:
    name = "base"

    def log(self, metrics: dict, step: int) -> None:
        raise NotImplementedError

    def finish(self) -> None:
        pass


class JsonlBackend(TrackingBackend):
    name = "jsonl"

    def __init__(self, path: str):
        os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
        self.path = path

    def log(self, metrics: dict, step: int) -> None:
        rec = {"step": step, "time": time.time()}
        rec.update({k: (float(v) if isinstance(v, (int, float)) else v) for k, v in metrics.items()
                    if isinstance(v, (int, float, str, bool)) or v is None})
        with open(self.path, "a") as f:
            f.write(json.dumps(rec) + "\n")


class CIHistoryBackend(JsonlBackend):
    """Per-run metric history consumed by CI gates (train/grad_norm, train/ppo_kl, rollout/raw_reward ...)."""
    name = "ci_history"


class DashboardBackend(TrackingBackend):
    """Feeds the run dashboard (``miles_b200/dashboard``): step metrics, trajectory life-cycle events and periodic
    read-only GPU samples go to its partitioned JSONL store."""
    name = "dashboard"

    # the part of the command line shown in the dashboard's header (written once to <root>/meta.json)
    SNAPSHOT_KEYS = ("wandb_group", "wandb_project", "colocate", "actor_num_nodes", "actor_num_gpus_per_node", "rollout_num_gpus",
                     "rollout_num_gpus_per_engine", "rollout_batch_size", "n_samples_per_prompt", "rollout_max_response_len",
                     "hf_checkpoint", "model_preset", "train_backend", "sglang_max_running_requests", "sglang_mem_fraction_static",
                     "use_miles_router", "tensor_model_parallel_size", "expert_model_parallel_size", "pipeline_model_parallel_size",
                     "context_parallel_size")

    def __init__(self, root: str, args=None, forward=None):
        import json

        from ..dashboard import Collector, EventStore
        from . import lifecycle

        self.root = root
        metrics = getattr(args, "dashboard_sglang_metrics", None)
        self.collector = Collector(EventStore(root), gpu_interval=float(getattr(args, "dashboard_gpu_sample_interval", None) or 5.0),
                                   engine_interval=getattr(args, "dashboard_sglang_scrape_interval", None),
                                   engine_metrics=[m.strip() for m in metrics.split(",") if m.strip()] if metrics else None,
                                   forward=forward)
        if args is not None:
            os.makedirs(root, exist_ok=True)
            with open(os.path.join(root, "meta.json"), "w") as f:
                json.dump({k: getattr(args, k) for k in self.SNAPSHOT_KEYS if getattr(args, k, None) is not None}, f, default=str)
            if getattr(args, "dashboard_sglang_scrape_mode", "auto") != "router":
                for u in [x for x in (getattr(args, "rollout_engine_urls", None) or "").split(",") if x]:
                    self.collector.add_engine(u)
            elif getattr(args, "rollout_router_url", None):
                self.collector.add_engine(args.rollout_router_url)
        lifecycle.add_sink(self.collector.on_lifecycle)
        self.collector.start()

    def log(self, metrics: dict, step: int) -> None:
        self.collector.log_metrics(metrics, step)

    def finish(self) -> None:
        self.collector.stop()


class WandbBackend(TrackingBackend):
    name = "wandb"

    def __init__(self, args):
        import wandb

        if getattr(args, "wandb_key", None):
            wandb.login(key=args.wandb_key, host=getattr(args, "wandb_host", None))
        name = getattr(args, "wandb_group", None)
        self.run = wandb.init(project=getattr(args, "wandb_project", None), entity=getattr(args, "wandb_team", None),
                              group=name, name=name, dir=getattr(args, "wandb_dir", None), id=getattr(args, "wandb_run_id", None),
                              mode=getattr(args, "wandb_mode", None), config={k: v for k, v in vars(args).items()
                                                                             if isinstance(v, (int, float, str, bool, type(None)))},
                              resume="allow")
        self.wandb = wandb

    def log(self, metrics: dict, step: int) -> None:
        self.wandb.log(metrics, step=step)

    def finish(self) -> None:
        self.wandb.finish()


class TensorboardBackend(TrackingBackend):
    name = "tensorboard"

    def __init__(self, args):
        from torch.utils.tensorboard import SummaryWriter

        d = os.path.join(os.environ.get("TENSORBOARD_DIR", "tensorboard"), getattr(args, "tb_project_name", None) or "miles_b200",
                         getattr(args, "tb_experiment_name", None) or time.strftime("%Y%m%d-%H%M%S"))
        self.w = SummaryWriter(d)

    def log(self, metrics: dict, step: int) -> None:
        for k, v in metrics.items():
            if isinstance(v, (int, float)):
                self.w.add_scalar(k, v, step)

    def finish(self) -> None:
        self.w.close()


class MlflowBackend(TrackingBackend):
    name = "mlflow"

    def __init__(self, args):
        import mlflow

        if getattr(args, "mlflow_tracking_uri", None):
            mlflow.set_tracking_uri(args.mlflow_tracking_uri)
        if getattr(args, "mlflow_experiment_name", None):
            mlflow.set_experiment(args.mlflow_experiment_name)
        mlflow.start_run(run_name=getattr(args, "mlflow_run_name", None), run_id=getattr(args, "mlflow_run_id", None))
        self.mlflow = mlflow

    def log(self, metrics: dict, step: int) -> None:
        self.mlflow.log_metrics({k.replace("@", "_at_"): float(v) for k, v in metrics.items() if isinstance(v, (int, float))}, step=step)

    def finish(self) -> None:
        self.mlflow.end_run()


class PrometheusBackend(TrackingBackend):
    name = "prometheus"

    def __init__(self, args):
        from prometheus_client import Gauge, start_http_server

        self.Gauge = Gauge
        self.gauges: dict = {}
        self.run = getattr(args, "prometheus_run_name", None) or "miles_b200"
        port = getattr(args, "prometheus_port", None)
        if port:
            start_http_server(int(port))

    def log(self, metrics: dict, step: int) -> None:
        for k, v in metrics.items():
            if not isinstance(v, (int, float)):
                continue
            name = "miles_" + "".join(c if c.isalnum() else "_" for c in k)
            g = self.gauges.get(name)
            if g is None:
                g = self.gauges[name] = self.Gauge(name, k, ["run"])
            g.labels(run=self.run).set(float(v))

    def set_gauge(self, name: str, value: float, labels: Optional[dict] = None) -> None:
        """A gauge that is not a step metric (the dashboard collector's GPU and engine samples,
        ``--dashboard-forward-prometheus``)."""
        name = "miles_" + "".join(c if c.isalnum() else "_" for c in name)
        keys = ["run"] + sorted(labels or {})
        g = self.gauges.get(name)
        if g is None:
            g = self.gauges[name] = self.Gauge(name, name, keys)
        g.labels(run=self.run, **{k: str(v) for k, v in (labels or {}).items()}).set(float(value))


class TrackingManager:
    def __init__(self, backends: Optional[list] = None):
        self.backends = backends or []
        self.history: list = []

    def log(self, metrics: dict, step: int) -> None:
        self.history.append((step, dict(metrics)))
        for b in self.backends:
            try:
                b.log(metrics, step)
            except Exception as e:  # noqa: BLE001 - a tracking outage must not stop training
                print(f"[tracking] backend {b.name} failed: {e}")

    def finish(self) -> None:
        for b in self.backends:
            b.finish()


def init_tracking(args, primary: bool = True) -> TrackingManager:
    if not primary:
        return TrackingManager([])
    backends = []
    for flag, cls in (("use_wandb", WandbBackend), ("use_tensorboard", TensorboardBackend), ("use_mlflow", MlflowBackend),
                      ("use_prometheus", PrometheusBackend)):
        if getattr(args, flag, False):
            try:
                backends.append(cls(args))
            except Exception as e:  # noqa: BLE001
                print(f"[tracking] {cls.name} disabled: {e}")
    if getattr(args, "use_miles_dashboard", False) and not getattr(args, "dump_details", None):
        raise ValueError("--use-miles-dashboard writes its telemetry under <dump-details>/dashboard: --dump-details is required")
    if getattr(args, "dump_details", None):
        forward = None
        if getattr(args, "dashboard_forward_prometheus", False):
            prom = next((b for b in backends if getattr(b, "name", "") == "prometheus"), None)
            if prom is not None and hasattr(prom, "set_gauge"):
                forward = prom.set_gauge
        backends.append(DashboardBackend(os.path.join(args.dump_details, "dashboard"), args, forward))
        backends.append(JsonlBackend(os.path.join(args.dump_details, "metrics.jsonl")))
    if os.environ.get("MILES_CI_HISTORY_PATH"):
        backends.append(CIHistoryBackend(os.environ["MILES_CI_HISTORY_PATH"]))
    return TrackingManager(backends)
