"""Single-turn generation: one request per sample; partially generated samples continue from their tokens
(reference: miles/rollout/generate_hub/single_turn.py:16-47)."""
from __future__ import annotations

from ...utils.types import Sample
from ..base_types import GenerateFnInput, GenerateFnOutput
from .common import compute_request_payload, prompt_ids, update_sample_from_response


async def generate(inp: GenerateFnInput) -> GenerateFnOutput:
    state, sample = inp.state, inp.sample
    sp = dict(inp.sampling_params)
    if sample.response_length > 0:  # partial rollout: continue after what was already generated
        ids = list(sample.tokens)
        sp["max_new_tokens"] = sp["max_new_tokens"] - sample.response_length
        if getattr(state.args, "mask_offpolicy_in_partial_rollout", False) and sample.loss_mask is None:
            sample.loss_mask = [0] * sample.response_length
    else:
        ids = prompt_ids(state, sample)
    payload = compute_request_payload(state, sample, ids, sp)
    if payload is None:
        sample.status = Sample.Status.TRUNCATED
        if not sample.tokens:
            sample.tokens = ids
        return GenerateFnOutput(samples=sample)
    out = await state.client.generate(payload)
    update_sample_from_response(state, sample, ids, out)
    return GenerateFnOutput(samples=sample)
