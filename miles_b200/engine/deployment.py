"""Deployment description of the rollout side: models, their server groups and the GPUs each engine gets.

A YAML file (``--sglang-config``) lists models; a model lists server groups of type ``regular``, ``prefill``,
``decode`` (prefill/decode disaggregation) or ``placeholder`` (GPUs reserved, no engine). Group settings override
model settings, which override the command line (``--rollout-num-gpus-per-engine``, ``--sglang-*`` passthrough).
Exactly the models whose path equals the trained checkpoint receive weight updates unless a model says otherwise;
every model gets its own router.

    sglang:
      - name: actor
        server_groups:
          - {worker_type: prefill, num_gpus: 2, num_gpus_per_engine: 1}
          - {worker_type: decode,  num_gpus: 4, num_gpus_per_engine: 2, overrides: {max_running_requests: 256}}
      - name: reward
        model_path: /ckpt/rm
        update_weights: false
        server_groups: [{worker_type: regular, num_gpus: 2}]

``plan()`` turns the description into a flat list of engine placements (model, group, worker type, GPU ids,
merged overrides) that the launcher walks.

Reference counterpart: miles/backends/sglang_utils/sglang_config.py:13-194 and the server-group bring-up in
miles/ray/rollout/rollout_server.py:17-301, miles/ray/rollout/server_group.py:24-274.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

WORKER_TYPES = ("regular", "prefill", "decode", "placeholder")


@dataclass
class ServerGroup:
    worker_type: str
    num_gpus: int
    num_gpus_per_engine: Optional[int] = None
    overrides: dict = field(default_factory=dict)

    def __post_init__(self):
        if self.worker_type not in WORKER_TYPES:
            raise ValueError(f"worker_type {self.worker_type!r} is not one of {WORKER_TYPES}")
        if self.num_gpus <= 0:
            raise ValueError("a server group needs at least one GPU")


@dataclass
class ModelDeployment:
    name: str
    model_path: Optional[str] = None
    num_gpus_per_engine: Optional[int] = None
    server_groups: list = field(default_factory=list)
    update_weights: Optional[bool] = None
    overrides: dict = field(default_factory=dict)

    def resolve(self, args) -> None:
        """Fill defaults from the command line and check the groups."""
        if self.model_path is None:
            self.model_path = getattr(args, "hf_checkpoint", None)
        if self.update_weights is None:
            self.update_weights = self.model_path == getattr(args, "hf_checkpoint", None)
        default_per_engine = self.num_gpus_per_engine or getattr(args, "rollout_num_gpus_per_engine", 1) or 1
        for g in self.server_groups:
            if g.num_gpus_per_engine is None:
                g.num_gpus_per_engine = default_per_engine
            if g.worker_type != "placeholder" and g.num_gpus % g.num_gpus_per_engine:
                raise ValueError(f"model {self.name}: {g.num_gpus} GPUs do not divide into engines of {g.num_gpus_per_engine}")
        kinds = {g.worker_type for g in self.server_groups}
        if ("prefill" in kinds) != ("decode" in kinds):
            raise ValueError(f"model {self.name}: prefill and decode groups come together")

    @property
    def has_pd_disaggregation(self) -> bool:
        return any(g.worker_type == "prefill" for g in self.server_groups)

    @property
    def total_num_gpus(self) -> int:
        return sum(g.num_gpus for g in self.server_groups)


@dataclass
class EnginePlacement:
    model: str
    group_index: int
    worker_type: str
    gpu_ids: list
    model_path: Optional[str]
    update_weights: bool
    overrides: dict


@dataclass
class Deployment:
    models: list = field(default_factory=list)

    @staticmethod
    def from_dict(d: dict) -> "Deployment":
        items = d.get("sglang", d.get("models", [])) if isinstance(d, dict) else d
        models = []
        for m in items:
            groups = [ServerGroup(**g) for g in m.get("server_groups", [])]
            models.append(ModelDeployment(m["name"], m.get("model_path"), m.get("num_gpus_per_engine"), groups,
                                          m.get("update_weights"), dict(m.get("overrides", {}))))
        names = [m.name for m in models]
        if len(set(names)) != len(names):
            raise ValueError(f"model names must be unique, got {names}")
        return Deployment(models)

    @staticmethod
    def from_yaml(path: str) -> "Deployment":
        import yaml

        with open(path) as f:
            return Deployment.from_dict(yaml.safe_load(f))

    @staticmethod
    def from_args(args) -> "Deployment":
        """The single-model deployment the plain flags describe: all rollout GPUs in one regular group, or a
        prefill/decode split when ``--prefill-num-servers`` is given."""
        per = getattr(args, "rollout_num_gpus_per_engine", 1) or 1
        total = getattr(args, "rollout_num_gpus", None) or per
        pre = getattr(args, "prefill_num_servers", None)
        if pre:
            groups = [ServerGroup("prefill", pre * per, per), ServerGroup("decode", total - pre * per, per)]
        else:
            groups = [ServerGroup("regular", total, per)]
        return Deployment([ModelDeployment("default", server_groups=groups)])

    def resolve(self, args) -> "Deployment":
        for m in self.models:
            m.resolve(args)
        if sum(bool(m.update_weights) for m in self.models) > 1:
            raise ValueError("only one model can receive weight updates from the trainer")
        return self

    @property
    def has_pd_disaggregation(self) -> bool:
        return any(m.has_pd_disaggregation for m in self.models)

    @property
    def total_num_gpus(self) -> int:
        return sum(m.total_num_gpus for m in self.models)

    def updatable_model(self) -> Optional[ModelDeployment]:
        return next((m for m in self.models if m.update_weights), None)

    def plan(self, first_gpu: int = 0) -> list:
        """Engine placements in GPU order; placeholder groups advance the GPU cursor without producing engines."""
        out, cur = [], first_gpu
        for m in self.models:
            for gi, g in enumerate(m.server_groups):
                if g.worker_type == "placeholder":
                    cur += g.num_gpus
                    continue
                for _ in range(g.num_gpus // g.num_gpus_per_engine):
                    ov = dict(m.overrides)
                    ov.update(g.overrides)
                    out.append(EnginePlacement(m.name, gi, g.worker_type, list(range(cur, cur + g.num_gpus_per_engine)),
                                               m.model_path, bool(m.update_weights), ov))
                    cur += g.num_gpus_per_engine
        return out
