"""Benchmark generate function: every sample is forced to a predetermined output length
(reference: miles/rollout/generate_hub/benchmarkers.py).  The length comes from
``sample.metadata['forced_length']`` or is drawn from a seeded log-normal clipped to
``[min_len, rollout_max_response_len]``; stop tokens are ignored so that synthetic random-weight models,
which never emit EOS, produce a realistic long-tailed length distribution."""
from __future__ import annotations

import math
import random

from ..base_types import GenerateFnInput, GenerateFnOutput
from .common import compute_request_payload, prompt_ids, update_sample_from_response


def forced_length_for(index: int, seed: int, mean: float, max_len: int, min_len: int = 16, sigma: float = 0.8) -> int:
    rng = random.Random(seed * 1000003 + index)
    mu = math.log(max(mean, 1.0)) - 0.5 * sigma * sigma
    return int(min(max(rng.lognormvariate(mu, sigma), min_len), max_len))


def add_arguments(parser) -> None:
    parser.add_argument("--benchmark-mean-response-len", type=float, default=None)
    parser.add_argument("--benchmark-response-sigma", type=float, default=0.8)


async def generate(inp: GenerateFnInput) -> GenerateFnOutput:
    state, sample = inp.state, inp.sample
    a = state.args
    sp = dict(inp.sampling_params)
    forced = (sample.metadata or {}).get("forced_length")
    if forced is None:
        mean = getattr(a, "benchmark_mean_response_len", None) or sp["max_new_tokens"] / 4
        forced = forced_length_for(sample.index or 0, a.rollout_seed, mean, sp["max_new_tokens"],
                                   sigma=getattr(a, "benchmark_response_sigma", 0.8))
    sp["forced_length"] = int(forced)
    sp["ignore_eos"] = True
    ids = prompt_ids(state, sample)
    payload = compute_request_payload(state, sample, ids, sp)
    out = await state.client.generate(payload)
    update_sample_from_response(state, sample, ids, out)
    return GenerateFnOutput(samples=sample)


generate.add_arguments = add_arguments
