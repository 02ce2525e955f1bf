"""Per-dataset evaluation settings: ``--eval-prompt-data name path [name path ...]`` gives the defaults, an
``--eval-config`` YAML may override them per dataset (samples per prompt, temperature, max response length, reward
type, generate function).

Reference: miles/utils/eval_config.py (208 lines).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional


@dataclass
class EvalDatasetConfig:
    name: str
    path: str
    n_samples_per_eval_prompt: int = 1
    temperature: Optional[float] = None
    top_p: Optional[float] = None
    top_k: Optional[int] = None
    max_response_len: Optional[int] = None
    rm_type: Optional[str] = None
    custom_generate_function_path: Optional[str] = None
    input_key: Optional[str] = None
    label_key: Optional[str] = None
    metadata_overrides: dict = field(default_factory=dict)

    def sampling_params(self, args) -> dict:
        pick = lambda v, *names: v if v is not None else next((getattr(args, n) for n in names if getattr(args, n, None) is not None), None)
        return {"temperature": pick(self.temperature, "eval_temperature", "rollout_temperature"),
                "top_p": pick(self.top_p, "eval_top_p", "rollout_top_p"), "top_k": pick(self.top_k, "eval_top_k", "rollout_top_k"),
                "max_new_tokens": pick(self.max_response_len, "eval_max_response_len", "rollout_max_response_len")}


def build_eval_configs(args) -> list:
    pairs = list(getattr(args, "eval_prompt_data", None) or [])
    assert len(pairs) % 2 == 0, "--eval-prompt-data takes name/path pairs"
    out = {pairs[i]: EvalDatasetConfig(pairs[i], pairs[i + 1], n_samples_per_eval_prompt=getattr(args, "n_samples_per_eval_prompt", 1) or 1)
           for i in range(0, len(pairs), 2)}
    path = getattr(args, "eval_config", None)
    if path:
        import yaml

        doc = yaml.safe_load(open(path)) or {}
        defaults = doc.get("defaults", {})
        for d in doc.get("datasets", []):
            base = out.get(d["name"], EvalDatasetConfig(d["name"], d.get("path", "")))
            for k, v in {**defaults, **d}.items():
                if k in EvalDatasetConfig.__dataclass_fields__:
                    setattr(base, k, v)
                else:
                    base.metadata_overrides[k] = v
            out[d["name"]] = base
    return list(out.values())
