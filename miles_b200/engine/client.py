"""Async client over one or more in-process engines: the ``/generate`` request/response contract.

Rollout code talks to engines through ``await client.generate(payload)`` exactly as the reference's
rollout functions POST to the router (miles/rollout/generate_utils/generate_endpoint_utils.py:52-140,
miles/router/router.py:215-230).  Requests are routed to the engine with the fewest in-flight requests;
a single pump task steps every engine while requests are outstanding, so generate functions, reward
models and the engine loop interleave cooperatively on one event loop without extra processes.
"""
from __future__ import annotations

import asyncio
import base64
import itertools
from typing import Optional, Sequence

import numpy as np
import torch

from .core import Engine, SamplingParams


class EngineClient:
    def __init__(self, engines: Sequence[Engine], tokenizer=None):
        self.engines = list(engines)
        self.tokenizer = tokenizer
        self._futures: dict = {}
        self._inflight = [0] * len(self.engines)
        self._owner: dict = {}
        self._pump_task: Optional[asyncio.Task] = None
        self._rid = itertools.count()
        self.lockstep_hook = None  # multi-rank engines: called once per pump iteration to keep ranks aligned

    # ------------------------------------------------------------------ routing
    def _pick(self) -> int:
        return min(range(len(self.engines)), key=lambda i: self._inflight[i])

    async def generate(self, payload: dict) -> dict:
        ids = payload.get("input_ids")
        if ids is None:
            assert self.tokenizer is not None, "text prompts need a tokenizer"
            ids = self.tokenizer(payload["text"], add_special_tokens=False)["input_ids"]
        if int((payload.get("sampling_params") or {}).get("max_new_tokens", 1) or 0) == 0:
            return self._score(ids, payload)
        sp = SamplingParams.from_dict(payload.get("sampling_params") or {})
        rid = payload.get("rid") or f"c{next(self._rid)}"
        i = self._pick()
        fut = asyncio.get_running_loop().create_future()
        self._futures[rid] = fut
        self._owner[rid] = i
        self._inflight[i] += 1
        self.engines[i].add_request(ids, sp, rid=rid, return_routed_experts=bool(payload.get("return_routed_experts")))
        self._ensure_pump()
        res = await fut
        meta = res["meta_info"]
        if "routed_experts" in meta and isinstance(meta["routed_experts"], torch.Tensor):
            arr = meta["routed_experts"].numpy().astype(np.int32)
            meta["routed_experts_shape"] = list(arr.shape)
            meta["routed_experts"] = base64.b64encode(arr.tobytes()).decode()
        if self.tokenizer is not None and not payload.get("skip_detokenize"):
            res["text"] = self.tokenizer.decode(res["output_ids"], skip_special_tokens=bool(
                (payload.get("sampling_params") or {}).get("skip_special_tokens", True)))
        else:
            res["text"] = ""
        return res

    def _score(self, ids: list, payload: dict) -> dict:
        """``max_new_tokens = 0``: score the input instead of generating (the request a distillation teacher gets,
        reference: miles/rollout/on_policy_distillation.py:104-125). ``meta_info.input_token_logprobs`` holds
        ``[logprob, token]`` per input token from ``logprob_start_len`` on (the first token of a sequence has none);
        ``top_logprobs_num = k`` adds ``input_top_logprobs``: per position the k ``[logprob, token]`` pairs."""
        start = int(payload.get("logprob_start_len", 0) or 0)
        k = int(payload.get("top_logprobs_num", 0) or 0)
        out = self.engines[self._pick()].score(ids, temperature=1.0, top_k=k)
        meta = {"prompt_tokens": len(ids), "completion_tokens": 0, "finish_reason": {"type": "length"},
                "input_token_logprobs": [[lp, t] for lp, t in zip(out["logprobs"], ids)][start:],
                "output_token_logprobs": [], "weight_version": self.engines[0].weight_version}
        if k:
            meta["input_top_logprobs"] = [None if tp is None else [[l, t] for l, t in zip(tp["logprobs"], tp["ids"])]
                                          for tp in out["top"]][start:]
        return {"output_ids": [], "text": "", "meta_info": meta}

    def _ensure_pump(self) -> None:
        if self._pump_task is None or self._pump_task.done():
            self._pump_task = asyncio.get_running_loop().create_task(self._pump())

    def _resolve(self, req) -> None:
        fut = self._futures.pop(req.rid, None)
        i = self._owner.pop(req.rid, None)
        if i is not None:
            self._inflight[i] -= 1
        if fut is not None and not fut.done():
            fut.set_result(req.result())

    async def _pump(self) -> None:
        while self._futures:
            progressed = False
            for e in self.engines:
                if e.sync is not None or (e.has_work() and not e.paused):
                    for req in e.step():
                        self._resolve(req)
                    progressed = True
                for req in e.pop_finished():
                    self._resolve(req)
            if self.lockstep_hook is not None:
                self.lockstep_hook()
            await asyncio.sleep(0 if progressed else 0.001)

    # ------------------------------------------------------------------ control plane
    async def abort_all(self) -> None:
        for e in self.engines:
            e.abort_request(abort_all=True)
            for req in e.pop_finished():
                self._resolve(req)

    def pause_generation(self, mode: str = "retract") -> None:
        for e in self.engines:
            e.pause_generation(mode)
            for req in e.pop_finished():
                self._resolve(req)

    def continue_generation(self) -> None:
        for e in self.engines:
            e.continue_generation()

    def weight_version(self) -> int:
        return self.engines[0].weight_version if self.engines else 0


def decode_routed_experts(meta: dict):
    """Inverse of the base64 transport used for ``routed_experts`` -> int32 array [T-1, L, K]."""
    raw = meta.get("routed_experts")
    if raw is None:
        return None
    if isinstance(raw, str):
        arr = np.frombuffer(base64.b64decode(raw), dtype=np.int32).copy()
        shp = meta.get("routed_experts_shape")
        return arr.reshape(shp) if shp else arr
    return np.asarray(raw, dtype=np.int32)
