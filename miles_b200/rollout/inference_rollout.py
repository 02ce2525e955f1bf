"""The default rollout function: generate groups until ``rollout_batch_size`` valid groups exist.

Behaviour of miles/rollout/inference_rollout/inference_rollout_train.py:86-185 in the reference:
over-sampling (``--over-sampling-batch-size`` groups are submitted at a time), dynamic filtering of
finished groups (e.g. non-zero reward std), aborting the leftovers once enough groups are collected,
recycling partially generated groups into the data-source buffer (``--partial-rollout``), and reward
computation per sample or per group (``--group-rm``).
"""
from __future__ import annotations

import asyncio
import time
from collections import Counter
from typing import Optional

from ..utils.misc import load_function
from ..utils.types import Sample
from .base_types import GenerateFnInput, RolloutFnConstructorInput, RolloutFnEvalOutput, RolloutFnTrainOutput
from .generate_hub.common import GenerateState
from .rm_hub import async_rm, batched_async_rm


def _resolve_generate_fn(args, sample: Optional[Sample] = None):
    path = (sample.generate_function_path if sample is not None and sample.generate_function_path else None) or \
        getattr(args, "custom_generate_function_path", None)
    if path:
        return load_function(path)
    from .generate_hub.single_turn import generate

    return generate


async def generate_and_rm(state: GenerateState, sample, sampling_params: dict, evaluation: bool = False):
    args = state.args
    if isinstance(sample, Sample) and sample.status in (Sample.Status.COMPLETED, Sample.Status.TRUNCATED) and sample.reward is not None:
        return sample
    if state.aborted:
        sample.status = Sample.Status.ABORTED
        return sample
    fn = _resolve_generate_fn(args, sample)
    try:
        out = await fn(GenerateFnInput(state, sample, dict(sampling_params), evaluation))
    finally:
        pacer = getattr(state, "pacer", None)
        if pacer is not None and not evaluation:
            pacer.sample_finished()  # --rollout-submission-granularity sample: this sample's slot is free again
    result = out.samples if hasattr(out, "samples") else out
    if getattr(args, "group_rm", False) and not evaluation:
        return result
    items = result if isinstance(result, list) else [result]
    opd = getattr(args, "use_opd", False) and getattr(args, "opd_type", None) == "sglang" and not evaluation
    if getattr(args, "recompute_logprobs_via_prefill", False) and not evaluation:
        from .generate_hub.prefill_logprobs import recompute_rollout_logprobs_via_prefill

        for s in items:
            await recompute_rollout_logprobs_via_prefill(args, state, s)
    for s in items:
        if opd and s.teacher_log_probs is None:
            # on-policy distillation against a teacher server: its log-probs of the sampled tokens travel with the sample
            from .on_policy_distillation import fetch_teacher_log_probs

            await fetch_teacher_log_probs(args, s, post=getattr(state, "teacher_post", None),
                                          vocab_size=getattr(getattr(state.client, "engines", [None])[0], "cfg", None).vocab_size
                                          if getattr(state.client, "engines", None) else None)
        if s.status == Sample.Status.ABORTED or s.reward is not None:
            continue
        if opd and getattr(args, "rm_type", None) is None and not getattr(args, "custom_rm_path", None):
            s.reward = 0.0  # pure distillation: the signal is the per-token penalty, there is no task reward
            continue
        s.reward = await async_rm(args, s)
    return result


async def generate_and_rm_group(state: GenerateState, group: list, sampling_params: dict, evaluation: bool = False) -> list:
    results = await asyncio.gather(*[generate_and_rm(state, s, sampling_params, evaluation) for s in group])
    flat = []
    for r in results:
        flat.extend(r if isinstance(r, list) else [r])
    if getattr(state.args, "group_rm", False) and not evaluation and not state.aborted:
        todo = [s for s in flat if s.status != Sample.Status.ABORTED]
        rewards = await batched_async_rm(state.args, todo)
        for s, r in zip(todo, rewards):
            s.reward = r
    return flat


class InferenceRolloutFn:
    """Class-based rollout function; one instance lives for the whole run."""

    def __init__(self, inp: RolloutFnConstructorInput):
        self.args = inp.args
        self.data_source = inp.data_source
        self.state = GenerateState(inp.args, inp.engine_client, getattr(inp.engine_client, "tokenizer", None))
        p = getattr(self.args, "dynamic_sampling_filter_path", None)
        self.dynamic_filter = load_function(p) if p else None
        p = getattr(self.args, "rollout_sample_filter_path", None)
        self.sample_filter = load_function(p) if p else None
        p = getattr(self.args, "rollout_all_samples_process_path", None)
        self.all_samples_process = load_function(p) if p else None

    async def __call__(self, inp):
        if inp.evaluation:
            return await self.eval_rollout(inp.rollout_id)
        return await self.generate_rollout_async(inp.rollout_id)

    async def generate_rollout_async(self, rollout_id: int) -> RolloutFnTrainOutput:
        args, state = self.args, self.state
        state.aborted = False
        target = args.rollout_batch_size
        data: list = []
        all_groups: list = []
        pending: set = set()
        drop_reasons: Counter = Counter()
        t0 = time.perf_counter()

        # pacing of the submissions (rollout/submission.py): by group (a slot frees when a whole prompt group is back) or by
        # sample (every finished sample frees its slot, so the engine's batch stays full behind a group's stragglers)
        from .submission import make_pacer

        pacer = state.pacer = make_pacer(args)

        def submit(n_groups: int) -> None:
            groups = self.data_source.get_samples(n_groups)
            pacer.submitted(groups)
            for group in groups:
                pending.add(asyncio.ensure_future(generate_and_rm_group(state, group, state.sampling_params)))

        while len(data) < target:
            if pacer.may_submit(len(pending), target - len(data)):
                submit(args.over_sampling_batch_size)
            if not pending:
                continue
            done, pending = await pacer.wait(pending)
            for task in done:
                group = task.result()
                all_groups.append(group)
                if any(s.status == Sample.Status.ABORTED for s in group):
                    continue
                if self.dynamic_filter is not None:
                    verdict = self.dynamic_filter(args, group)
                    keep = verdict.keep if hasattr(verdict, "keep") else bool(verdict)
                    if not keep:
                        drop_reasons[getattr(verdict, "reason", None) or "filtered"] += 1
                        continue
                if len(data) < target:
                    data.append(group)
        aborted = await self._abort(pending)
        if getattr(args, "partial_rollout", False) and aborted:
            self.data_source.add_samples(aborted)
        data.sort(key=lambda g: g[0].index if g and g[0].index is not None else 0)
        if self.sample_filter is not None:
            self.sample_filter(args, data)
        if self.all_samples_process is not None:
            self.all_samples_process(args, all_groups, self.data_source)
        metrics = {"rollout/dynamic_filter/drop_" + k: v for k, v in drop_reasons.items()}
        metrics["perf/rollout_generate_time"] = time.perf_counter() - t0
        return RolloutFnTrainOutput(samples=data, metrics=metrics)

    async def _abort(self, pending: set) -> list:
        """Abort in-flight requests; return the partially generated groups (for partial rollout)."""
        if not pending:
            return []
        self.state.aborted = True
        await self.state.client.abort_all()
        groups = []
        for task in pending:
            try:
                group = await task
            except Exception:
                continue
            if any(s.response_length > 0 for s in group):
                for s in group:
                    if s.status == Sample.Status.ABORTED:
                        s.reward = None
                groups.append(group)
        self.state.aborted = False
        return groups

    async def eval_rollout(self, rollout_id: int) -> RolloutFnEvalOutput:
        from .eval import eval_rollout

        return await eval_rollout(self.args, self.state, rollout_id)


def run_rollout_fn(fn, inp):
    """Drive a (possibly async) rollout function to completion from synchronous code."""
    out = fn(inp)
    if asyncio.iscoroutine(out):
        out = asyncio.run(out)
    if isinstance(out, (RolloutFnTrainOutput, RolloutFnEvalOutput)):
        return out
    return RolloutFnEvalOutput(data=out) if inp.evaluation else RolloutFnTrainOutput(samples=out)
