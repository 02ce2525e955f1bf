"""``Sample`` — the unit of rollout data exchanged between data source, generate functions, reward
functions and the trainer (field set of the reference's miles/utils/types.py:25-297)."""
from __future__ import annotations

import copy
from dataclasses import dataclass, field, fields
from enum import Enum
from typing import Any, Optional


@dataclass
class Sample:
    group_index: Optional[int] = None
    index: Optional[int] = None
    rollout_id: Optional[int] = None      # siblings of one trajectory share it; None -> ``index``
    prompt: Any = ""                      # text or chat messages
    tokens: list = field(default_factory=list)        # prompt + response token ids
    multimodal_inputs: Optional[dict] = None
    multimodal_train_inputs: Optional[dict] = None
    response: str = ""
    response_length: int = 0
    label: Optional[Any] = None
    reward: Any = None                    # float or dict (see --reward-key)
    loss_mask: Optional[list] = None      # over the response; None = all ones
    weight_versions: list = field(default_factory=list)
    rollout_log_probs: Optional[list] = None
    rollout_routed_experts: Any = None    # int32 [num_tokens-1, num_moe_layers, top_k]
    rollout_indexer_topk: Any = None
    remove_sample: bool = False
    teacher_log_probs: Optional[list] = None
    opd_reverse_kl: Optional[list] = None

    class Status(Enum):
        PENDING = "pending"
        COMPLETED = "completed"
        TRUNCATED = "truncated"
        ABORTED = "aborted"
        FAILED = "failed"

    status: "Sample.Status" = None
    metadata: dict = field(default_factory=dict)
    generate_function_path: Optional[str] = None
    train_metadata: Optional[dict] = None
    adapter: Any = None
    reward_spec: Any = None
    routing_key: Optional[str] = None
    non_generation_time: float = 0.0
    spec_info: dict = field(default_factory=dict)
    prefix_cache_info: dict = field(default_factory=dict)

    def __post_init__(self):
        if self.status is None:
            self.status = Sample.Status.PENDING

    @property
    def effective_rollout_id(self) -> int:
        return self.rollout_id if self.rollout_id is not None else self.index

    @property
    def prompt_length(self) -> int:
        return len(self.tokens) - self.response_length

    def get_reward_value(self, key: Optional[str] = None) -> float:
        if isinstance(self.reward, dict):
            return float(self.reward[key] if key else next(iter(self.reward.values())))
        return float(self.reward)

    def oldest_weight_version(self) -> Optional[int]:
        vs = [int(v) for v in self.weight_versions if v is not None]
        return min(vs) if vs else None

    def to_dict(self) -> dict:
        d = {}
        for f in fields(self):
            v = getattr(self, f.name)
            if f.name == "status":
                v = v.value
            elif hasattr(v, "tolist") and not isinstance(v, list):
                v = v.tolist()
            d[f.name] = v
        return d

    @classmethod
    def from_dict(cls, d: dict) -> "Sample":
        d = dict(d)
        st = d.pop("status", "pending")
        names = {f.name for f in fields(cls)}
        s = cls(**{k: v for k, v in d.items() if k in names})
        s.status = st if isinstance(st, Sample.Status) else Sample.Status(st)
        return s

    def clone(self) -> "Sample":
        return copy.deepcopy(self)
