"""Contracts of the pluggable rollout layer (reference: miles/rollout/base_types.py:14-97).

* rollout function  : ``fn(RolloutFnTrainInput | RolloutFnEvalInput) -> RolloutFnTrainOutput | RolloutFnEvalOutput``
  (a class with ``__call__`` or a plain function, sync or async);
* generate function : ``async generate(GenerateFnInput) -> GenerateFnOutput`` producing one finished sample
  (or a list of samples for multi-sample trajectories).
"""
from __future__ import annotations

import asyncio
import inspect
from dataclasses import dataclass, field
from typing import Any


@dataclass
class RolloutFnConstructorInput:
    args: Any
    data_source: Any
    engine_client: Any = None


@dataclass
class RolloutFnTrainInput:
    rollout_id: int
    evaluation: bool = False


@dataclass
class RolloutFnEvalInput:
    rollout_id: int
    evaluation: bool = True


@dataclass
class RolloutFnTrainOutput:
    samples: list                      # list of groups (list[list[Sample]])
    metrics: dict = field(default_factory=dict)


@dataclass
class RolloutFnEvalOutput:
    data: dict                         # dataset name -> {"rewards": [...], "truncated": [...], "samples": [...]}
    metrics: dict = field(default_factory=dict)


@dataclass
class GenerateFnInput:
    state: Any                         # GenerateState: engine client, tokenizer, args, semaphore
    sample: Any
    sampling_params: dict
    evaluation: bool = False

    @property
    def args(self):
        return self.state.args


@dataclass
class GenerateFnOutput:
    samples: Any                       # Sample | list[Sample]


def call_rollout_fn(fn, inp):
    """Call a sync or async rollout function and normalise legacy return types."""
    out = fn(inp)
    if inspect.isawaitable(out):
        try:
            loop = asyncio.get_running_loop()
        except RuntimeError:
            loop = None
        if loop is not None and loop.is_running():
            raise RuntimeError("call_rollout_fn must not be invoked from a running event loop; await the function instead")
        out = asyncio.run(out)
    if isinstance(out, (RolloutFnTrainOutput, RolloutFnEvalOutput)):
        return out
    if inp.evaluation:
        return RolloutFnEvalOutput(data=out)
    return RolloutFnTrainOutput(samples=out)
