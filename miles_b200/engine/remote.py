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
    def __init__(self, urls: Sequence[str], tokenizer=None, transport=None, max_retries: int = 3):
        self.urls = [u.rstrip("/") for u in urls]
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
            return await http_utils.post(url + "/generate", payload, max_retries=self._retries, transport=self._transport)
        finally:
            self.inflight[url] -= 1

    # ------------------------------------------------------------------ control plane (all engines)
    async def _all(self, path: str, payload: Optional[dict] = None, method: str = "POST") -> list:
        return await asyncio.gather(*[http_utils.request(method, u + path, payload, max_retries=self._retries,
                                                         transport=self._transport) for u in self.urls])

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
