"""Request building and response folding shared by the generate functions
(reference: miles/rollout/generate_utils/generate_endpoint_utils.py:17-140)."""
from __future__ import annotations

from typing import Optional

from ...engine.client import decode_routed_experts
from ...utils.types import Sample


class GenerateState:
    """Per-run shared state of the generate functions: args, tokenizer, engine client, default sampling params."""

    def __init__(self, args, client, tokenizer=None):
        self.args = args
        self.client = client
        self.tokenizer = tokenizer
        self.sampling_params = dict(
            temperature=args.rollout_temperature, top_p=args.rollout_top_p, top_k=args.rollout_top_k,
            max_new_tokens=args.rollout_max_response_len, stop_token_ids=list(args.rollout_stop_token_ids or []),
            skip_special_tokens=getattr(args, "rollout_skip_special_tokens", False),
        )
        # --rollout-stop: stop words. A word that is one token becomes a stop token id (the engine stops on it); a longer
        # one is matched on the decoded response afterwards and the response is cut after its first occurrence.
        self.stop_strings: list = []
        for word in (getattr(args, "rollout_stop", None) or []):
            ids = tokenizer.encode(word, add_special_tokens=False) if tokenizer is not None else []
            if len(ids) == 1:
                self.sampling_params["stop_token_ids"].append(int(ids[0]))
            else:
                assert tokenizer is not None, "--rollout-stop with words needs a tokenizer (--hf-checkpoint); use --rollout-stop-token-ids"
                self.stop_strings.append(word)
        self.aborted = False

    def eval_sampling_params(self) -> dict:
        a = self.args
        sp = dict(self.sampling_params)
        for k, attr in (("temperature", "eval_temperature"), ("top_p", "eval_top_p"), ("top_k", "eval_top_k"),
                        ("max_new_tokens", "eval_max_response_len")):
            v = getattr(a, attr, None)
            if v is not None:
                sp[k] = v
        if getattr(a, "eval_min_new_tokens", None):
            sp["min_new_tokens"] = a.eval_min_new_tokens
        return sp


def prompt_ids(state: GenerateState, sample: Sample) -> list:
    if sample.tokens and sample.response_length == 0:
        return list(sample.tokens)
    if isinstance(sample.prompt, list) and sample.prompt and isinstance(sample.prompt[0], int):
        return list(sample.prompt)
    assert state.tokenizer is not None, "text prompts need a tokenizer (--hf-checkpoint)"
    return state.tokenizer(sample.prompt, add_special_tokens=False)["input_ids"]


def compute_request_payload(state: GenerateState, sample: Sample, input_ids: list, sampling_params: dict) -> Optional[dict]:
    """Builds the /generate payload; returns None when the context budget is already exhausted."""
    a = state.args
    sp = dict(sampling_params)
    max_ctx = getattr(a, "rollout_max_context_len", None)
    if max_ctx is not None:
        room = max_ctx - len(input_ids)
        if room <= 0:
            return None
        sp["max_new_tokens"] = min(sp.get("max_new_tokens", room), room)
    if sp.get("max_new_tokens", 1) <= 0:
        return None
    payload = {"input_ids": input_ids, "sampling_params": sp, "return_logprob": True}
    if getattr(a, "use_rollout_routing_replay", False):
        payload["return_routed_experts"] = True
    if sample.routing_key:
        payload["routing_key"] = sample.routing_key
    return payload


def update_sample_from_response(state: GenerateState, sample: Sample, input_ids: list, output: dict,
                                loss_mask_value: int = 1) -> Sample:
    meta = output["meta_info"]
    new_ids = list(output["output_ids"])
    lps = [lp for lp, _ in meta.get("output_token_logprobs", [])]
    if getattr(state, "stop_strings", None) and state.tokenizer is not None and new_ids:
        # cut after the first stop word: the shortest token prefix whose decoding contains it
        text = state.tokenizer.decode(new_ids, skip_special_tokens=False)
        hit = min((text.find(w) + len(w) for w in state.stop_strings if w in text), default=-1)
        if hit >= 0:
            k = next((k for k in range(1, len(new_ids) + 1)
                      if len(state.tokenizer.decode(new_ids[:k], skip_special_tokens=False)) >= hit), len(new_ids))
            new_ids, lps = new_ids[:k], lps[:k]
            output = dict(output, text=state.tokenizer.decode(new_ids, skip_special_tokens=True))
            meta = dict(meta, finish_reason={"type": "stop"})
    if not sample.tokens or sample.response_length == 0:
        sample.tokens = list(input_ids)
    sample.tokens = sample.tokens + new_ids
    sample.response_length += len(new_ids)
    sample.response = (sample.response or "") + (output.get("text") or "")
    sample.rollout_log_probs = (sample.rollout_log_probs or []) + lps
    if sample.loss_mask is not None or loss_mask_value != 1:
        sample.loss_mask = (sample.loss_mask or []) + [loss_mask_value] * len(new_ids)
    re = decode_routed_experts(meta)
    if re is not None:
        sample.rollout_routed_experts = re
    for v in meta.get("weight_versions", [meta.get("weight_version")]):
        if v is not None and (not sample.weight_versions or sample.weight_versions[-1] != v):
            sample.weight_versions.append(v)
    sample.prefix_cache_info = {"cached_tokens": sample.prefix_cache_info.get("cached_tokens", 0) + meta.get("cached_tokens", 0),
                                "total_prompt_tokens": sample.prefix_cache_info.get("total_prompt_tokens", 0) + meta.get("prompt_tokens", 0)}
    fr = meta["finish_reason"]["type"]
    sample.status = {"length": Sample.Status.TRUNCATED, "abort": Sample.Status.ABORTED}.get(fr, Sample.Status.COMPLETED)
    return sample
