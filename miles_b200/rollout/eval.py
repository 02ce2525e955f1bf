"""Evaluation rollouts: per-dataset configs, generation with eval sampling params, reward statistics.

Datasets come from ``--eval-prompt-data name path [name path ...]`` or a YAML ``--eval-config`` whose
entries may override ``n_samples_per_eval_prompt, temperature, top_p, top_k, max_response_len, rm_type,
input_key, label_key`` (reference: miles/utils/eval_config.py and
miles/rollout/inference_rollout/inference_rollout_eval.py).
"""
from __future__ import annotations

import asyncio
import copy
from dataclasses import dataclass, field
from typing import Optional

from ..utils.types import Sample
from .base_types import RolloutFnEvalOutput


@dataclass
class EvalDatasetConfig:
    name: str
    path: str
    n_samples_per_eval_prompt: Optional[int] = None
    temperature: Optional[float] = None
    top_p: Optional[float] = None
    top_k: Optional[int] = None
    max_response_len: Optional[int] = None
    rm_type: Optional[str] = None
    input_key: Optional[str] = None
    label_key: Optional[str] = None
    metadata_key: Optional[str] = None
    custom_generate_function_path: Optional[str] = None
    extra: dict = field(default_factory=dict)


def resolve_eval_datasets(args) -> list:
    out = []
    cfg_path = getattr(args, "eval_config", None)
    if cfg_path:
        import yaml

        with open(cfg_path) as f:
            doc = yaml.safe_load(f) or {}
        defaults = (doc.get("eval") or {}).get("defaults", {})
        for d in (doc.get("eval") or {}).get("datasets", doc.get("datasets", [])):
            merged = {**defaults, **d}
            known = {k: merged.pop(k) for k in list(merged) if k in EvalDatasetConfig.__dataclass_fields__}
            out.append(EvalDatasetConfig(**known, extra=merged))
    pd = getattr(args, "eval_prompt_data", None)
    if pd:
        assert len(pd) % 2 == 0, "--eval-prompt-data takes name/path pairs"
        for i in range(0, len(pd), 2):
            out.append(EvalDatasetConfig(name=pd[i], path=pd[i + 1]))
    return out


async def eval_rollout(args, state, rollout_id: int) -> RolloutFnEvalOutput:
    from .data_source import Dataset
    from .inference_rollout import generate_and_rm

    data, metrics = {}, {}
    for ds in resolve_eval_datasets(args):
        local = copy.copy(args)
        if ds.rm_type:
            local.rm_type = ds.rm_type
        if ds.custom_generate_function_path:
            local.custom_generate_function_path = ds.custom_generate_function_path
        sub_state = copy.copy(state)
        sub_state.args = local
        dataset = Dataset(ds.path, state.tokenizer, getattr(args, "eval_max_prompt_len", None),
                          ds.input_key or getattr(args, "eval_input_key", None) or args.input_key,
                          ds.label_key or getattr(args, "eval_label_key", None) or args.label_key,
                          ds.metadata_key or args.metadata_key, getattr(args, "eval_tool_key", None) or getattr(args, "tool_key", None),
                          args.apply_chat_template, getattr(args, "apply_chat_template_kwargs", None))
        sp = state.eval_sampling_params()
        for k, attr in (("temperature", "temperature"), ("top_p", "top_p"), ("top_k", "top_k"), ("max_new_tokens", "max_response_len")):
            if getattr(ds, attr) is not None:
                sp[k] = getattr(ds, attr)
        n = ds.n_samples_per_eval_prompt or getattr(args, "n_samples_per_eval_prompt", 1) or 1
        tasks, idx = [], 0
        for i in range(len(dataset)):
            for _ in range(n):
                s = copy.deepcopy(dataset[i])
                s.group_index, s.index = i, idx
                idx += 1
                tasks.append(generate_and_rm(sub_state, s, sp, evaluation=True))
        samples = await asyncio.gather(*tasks)
        flat = []
        for s in samples:
            flat.extend(s if isinstance(s, list) else [s])
        key = getattr(args, "eval_reward_key", None)
        rewards = [s.get_reward_value(key) for s in flat if s.reward is not None]
        data[ds.name] = {"rewards": rewards, "truncated": [s.status == Sample.Status.TRUNCATED for s in flat], "samples": flat}
        if rewards:
            metrics[f"eval/{ds.name}"] = sum(rewards) / len(rewards)
            metrics[f"eval/{ds.name}-truncated_ratio"] = sum(data[ds.name]["truncated"]) / len(flat)
            metrics[f"eval/{ds.name}-response_len/mean"] = sum(s.response_length for s in flat) / len(flat)
    return RolloutFnEvalOutput(data=data, metrics=metrics)
