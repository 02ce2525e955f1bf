"""Client of rollout engines that live in other processes (`engine/server.py`), with the interface of the in-process
``EngineClient`` so that rollout and generate functions do not care where the engine runs.

Requests go to the engine with the fewest requests in flight (or to one router URL that balances itself); the
control calls fan out to every engine. Together with ``weight_sync.broadcast.BroadcastWeightUpdater`` and
``engine.deployment`` this is the disaggregated mode: trainer GPUs and rollout GPUs are different processes.

Reference counterpart: the HTTP path of miles/rollout/sglang_rollout.py:86-277 and the RPC methods of
miles/backends/sglang_utils/sglang_engine.py:126-693.
"""
from __future__ import annotations

import asyncio
import zlib
from typing import Optional, Sequence

from ..utils import http_utils


class RemoteEngineClient:
    def __init__(self, urls: Sequence[str], tokenizer=None, transport=None, max_retries: int = 3,
                 prefill_urls: Sequence[str] = ()):
        """``prefill_urls``: prefill / decode disaggregation. Those engines only prefill; ``urls`` minus them decode, and
        every request's prompt pages are handed from one to the other before it is submitted (engine/pd.py)."""
        self.prefill_urls = [u.rstrip("/") for u in prefill_urls]
        self.all_urls = [u.rstrip("/") for u in urls]
        self.urls = [u for u in self.all_urls if u not in self.prefill_urls]  # the engines that answer /generate
        self._prefill_rr = 0
        self.transferred_tokens = 0
        if not self.urls:
            raise ValueError("at least one engine URL is required")
        self.tokenizer = tokenizer
        self.inflight = {u: 0 for u in self.urls}
        self._transport, self._retries = transport, max_retries
        self._rr = 0

    # ------------------------------------------------------------------ data plane
    def _pick(self, routing_key: Optional[str] = None) -> str:
        if routing_key is not None:  # requests of one session stay on one engine (its KV cache holds their prefix)
            return self.urls[zlib.crc32(str(routing_key).encode()) % len(self.urls)]  # the same engine from any process
        low = min(self.inflight.values())
        cands = [u for u in self.urls if self.inflight[u] == low]
        self._rr += 1
        return cands[self._rr % len(cands)]

    async def generate(self, payload: dict) -> dict:
        if "input_ids" not in payload and "text" in payload and self.tokenizer is not None:
            payload = dict(payload, input_ids=self.tokenizer(payload["text"], add_special_tokens=False)["input_ids"])
        url = self._pick(payload.get("routing_key"))
        self.inflight[url] += 1
        try:
            if self.prefill_urls and "input_ids" in payload:
                await self._hand_over(payload, url)
            return await http_utils.post(url + "/generate", payload, max_retries=self._retries, transport=self._transport)
        finally:
            self.inflight[url] -= 1

    async def _hand_over(self, payload: dict, decode_url: str) -> None:
        """Prefill the prompt on a prefill engine and move its cached pages into the decode engine's prefix cache. A
        failure here costs only the saving: the decode engine then prefills the whole prompt itself."""
        from .pd import PDClient

        self._prefill_rr += 1
        pu = self.prefill_urls[self._prefill_rr % len(self.prefill_urls)]
        try:
            pd = PDClient([pu], [decode_url], transport=self._transport)
            warm = {"input_ids": payload["input_ids"], "return_logprob": False,
                    "sampling_params": {"max_new_tokens": 1, "temperature": 0.0, "ignore_eos": True},
                    "return_routed_experts": bool(payload.get("return_routed_experts"))}
            await pd._call(pu + "/generate", warm)
            blob = await pd._call(pu + "/export_prefix", {"input_ids": payload["input_ids"]}, raw=True)
            got = await pd._call(decode_url + "/import_prefix", blob)
            if isinstance(got, dict):
                self.transferred_tokens += int(got.get("cached_tokens", 0))
        except Exception:  # noqa: BLE001 - the request itself still runs
            pass

    # ------------------------------------------------------------------ control plane (all engines)
    async def _all(self, path: str, payload: Optional[dict] = None, method: str = "POST") -> list:
        targets = self.all_urls if getattr(self, "all_urls", None) else self.urls
        return await asyncio.gather(*[http_utils.request(method, u + path, payload, max_retries=self._retries,
                                                         transport=self._transport) for u in targets])

    async def abort_all(self) -> None:
        await self._all("/abort_request", {"abort_all": True})

    async def pause_generation(self, mode: str = "retract") -> None:
        await self._all("/pause_generation", {"mode": mode})

    async def continue_generation(self) -> None:
        await self._all("/continue_generation", {})

    async def flush_cache(self) -> None:
        await self._all("/flush_cache", {})

    async def weight_versions(self) -> list:
        return [r["weight_version"] for r in await self._all("/get_weight_version", None, "GET")]

    async def health(self) -> dict:
        """url -> True / False (one failing engine does not hide the others)."""
        async def one(u):
            try:
                r = await http_utils.get(u + "/health_generate", max_retries=0, transport=self._transport)
                return u, (r or {}).get("status") == "ok"
            except Exception:
                return u, False

        return dict(await asyncio.gather(*[one(u) for u in self.urls]))
