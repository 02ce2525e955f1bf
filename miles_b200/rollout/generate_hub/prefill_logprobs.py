"""``--recompute-logprobs-via-prefill``: after a sample is generated, its rollout log-probs are replaced by the ones the
engine computes in one prefill pass over the whole sequence (``/generate`` with ``max_new_tokens = 0``). Decode steps
and prefill run different kernels (split-KV decode attention, few-row weight streaming); the training forward is a
prefill, so log-probs recomputed this way differ from the trainer's by less than the ones recorded while decoding.

Reference: miles/rollout/generate_utils/prefill_logprobs.py:24-146.
"""
from __future__ import annotations

from ...utils.types import Sample


def scoring_payload(sample: Sample) -> dict:
    prompt_len = len(sample.tokens) - sample.response_length
    if prompt_len <= 0:
        raise ValueError(f"cannot score a response without a prompt token: tokens={len(sample.tokens)}, response_length={sample.response_length}")
    # entries come aligned to the input tokens from logprob_start_len on, the first without a value: start one token
    # before the response so that the tail holds every response token
    return {"input_ids": list(sample.tokens), "sampling_params": {"max_new_tokens": 0, "temperature": 0, "skip_special_tokens": False},
            "return_logprob": True, "logprob_start_len": prompt_len - 1}


def response_logprobs(sample: Sample, meta: dict) -> list:
    n = sample.response_length
    items = (meta.get("input_token_logprobs") or [])[-n:]
    want = list(sample.tokens[len(sample.tokens) - n:])
    got = [int(it[1]) for it in items]
    if got != want:
        raise ValueError(f"prefill scoring does not line up with the response: expected {want[:8]}... ({len(want)}), got {got[:8]}... ({len(got)})")
    lps = [it[0] for it in items]
    if any(lp is None for lp in lps):
        raise ValueError("prefill scoring returned no value for a response token")
    return [float(lp) for lp in lps]


async def recompute_rollout_logprobs_via_prefill(args, state, sample: Sample) -> None:
    if not getattr(args, "recompute_logprobs_via_prefill", False) or sample.status == Sample.Status.ABORTED:
        return
    if sample.response_length == 0:
        sample.rollout_log_probs = []
        return
    out = await state.client.generate(scoring_payload(sample))
    sample.rollout_log_probs = response_logprobs(sample, out["meta_info"])
    sample.metadata = dict(sample.metadata or {}, rollout_log_probs_source="prefill_recompute")
