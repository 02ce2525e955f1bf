"""On-policy distillation against teacher *servers* (``--use-opd --opd-type sglang``).

After a sample is generated its whole token sequence is sent to a teacher's scoring endpoint (``/generate`` with
``max_new_tokens = 0``, ``return_logprob``, ``logprob_start_len = 0``); the teacher's log-probs of the response tokens
become ``sample.teacher_log_probs``, which the trainer turns into the per-token penalty
``adv -= opd_kl_coef * (student_logprob - teacher_logprob)`` (``rl/advantages.py``, ``rl/opd.py``).

* one teacher: ``--rm-url http://teacher:port/generate``;
* several: ``--opd-teacher-urls NAME=URL ...`` and the sample's ``metadata[--opd-teacher-key]`` names its teacher
  (unknown or missing names go to the entry called ``default``, and fail if there is none: distilling from the wrong
  teacher silently would be worse than stopping);
* ``--opd-log-prob-top-k k``: the teacher returns only its k most likely tokens per position; a sampled token outside
  them gets the floor ``log(remaining mass / (V - k))`` (``rl/opd.py:teacher_logprob_from_topk``).

Reference: miles/rollout/on_policy_distillation.py:25-125, 281-436.
"""
from __future__ import annotations

from typing import Iterable, Optional

from ..rl.opd import teacher_logprob_from_topk
from ..utils.types import Sample

DEFAULT_TEACHER_NAME = "default"


def parse_teacher_urls(values: Optional[Iterable[str]]) -> dict:
    """``NAME=URL`` entries -> {name: url}; splits at the first ``=`` (URLs may contain more), rejects malformed and
    duplicate entries at start-up."""
    out: dict = {}
    for value in values or []:
        name, sep, url = value.partition("=")
        name, url = name.strip(), url.strip()
        if not sep or not name or not url:
            raise ValueError(f"invalid --opd-teacher-urls entry {value!r}: expected NAME=URL")
        if name in out:
            raise ValueError(f"duplicate teacher name {name!r} in --opd-teacher-urls")
        out[name] = url
    return out


def teacher_url_for_sample(args, sample: Sample) -> str:
    urls = parse_teacher_urls(getattr(args, "opd_teacher_urls", None))
    if not urls:
        assert getattr(args, "rm_url", None), "--opd-type sglang needs --rm-url or --opd-teacher-urls"
        return args.rm_url
    key = getattr(args, "opd_teacher_key", None) or "opd_teacher"
    name = (sample.metadata or {}).get(key) if isinstance(sample.metadata, dict) else None
    if name is not None and str(name) in urls:
        return urls[str(name)]
    if DEFAULT_TEACHER_NAME in urls:
        return urls[DEFAULT_TEACHER_NAME]
    raise ValueError(f"sample metadata[{key!r}]={name!r} names no teacher of --opd-teacher-urls ({sorted(urls)}) and there is "
                     f"no '{DEFAULT_TEACHER_NAME}' entry")


def score_payload(input_ids: list, top_k: int = 0) -> dict:
    p = {"input_ids": list(input_ids), "sampling_params": {"temperature": 0, "max_new_tokens": 0, "skip_special_tokens": False},
         "return_logprob": True, "logprob_start_len": 0}
    if top_k > 0:
        p["top_logprobs_num"] = top_k
    return p


def teacher_log_probs_from_response(sample: Sample, meta: dict, top_k: int, vocab_size: int) -> list:
    """Log-probs of the sample's response tokens out of a scoring response (aligned with ``logprob_start_len = 0``: entry
    ``i`` scores input token ``i``)."""
    n = sample.response_length
    toks = list(sample.tokens[len(sample.tokens) - n:]) if n else []
    if top_k > 0 and meta.get("input_top_logprobs") is not None:
        tops = meta["input_top_logprobs"][-n:] if n else []
        out = []
        for t, tp in zip(toks, tops):
            ids, lps = [int(e[1]) for e in (tp or [])], [float(e[0]) for e in (tp or [])]
            out.append(teacher_logprob_from_topk(t, ids, lps, vocab_size))
        return out
    entries = meta["input_token_logprobs"][-n:] if n else []
    assert len(entries) == n and all(int(e[1]) == int(t) for e, t in zip(entries, toks)), \
        "the teacher's scored tokens do not line up with the sample's response tokens"
    return [float(e[0]) for e in entries]


async def fetch_teacher_log_probs(args, sample: Sample, post=None, vocab_size: Optional[int] = None) -> Sample:
    """Fill ``sample.teacher_log_probs``. ``post(url, payload) -> dict`` defaults to an HTTP POST."""
    if sample.status == Sample.Status.ABORTED or not sample.response_length:
        sample.teacher_log_probs = [0.0] * int(sample.response_length or 0)
        return sample
    if post is None:
        from ..utils.http_utils import post as post
    top_k = max(0, int(getattr(args, "opd_log_prob_top_k", 0) or 0))
    out = await post(teacher_url_for_sample(args, sample), score_payload(sample.tokens, top_k))
    sample.teacher_log_probs = teacher_log_probs_from_response(sample, out["meta_info"], top_k, vocab_size or getattr(args, "vocab_size", None) or 0)
    return sample
