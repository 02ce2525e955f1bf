"""Prefill / decode disaggregation: prompts are prefilled on one group of engines, their keys / values travel to the
engine that decodes.

The hand-over is built on the prefix cache. A prefill engine runs the prompt (one forward, no decoding worth the
name), after which the prompt's full pages sit in its prefix cache; ``export_prefix`` reads them out, ``import_prefix``
on the decode engine writes them into freshly allocated pages and registers them in *its* prefix cache. The request
itself is then submitted to the decode engine unchanged: its prefill finds the imported pages and computes only the
tail (less than one page plus one token), and sampling, stop conditions, log-probs and routed experts are the decode
engine's own, so a disaggregated run returns what the decode engine alone would have returned. Keys / values computed
under another weight version are refused by the importer.

Transports: the same process (``PDPair``: tensors stay on the device) and HTTP (``PDClient``: ``/export_prefix`` on the
prefill engine returns one binary blob, ``/import_prefix`` on the decode engine takes it). Engines of one node could
pass CUDA-IPC handles instead of bytes; that form is not built.

Reference: the reference configures SGLang's prefill / decode server groups and its router's PD mode
(miles/backends/sglang_utils/sglang_config.py:13-194, miles/ray/rollout/rollout_server.py:17-301); the transfer itself
is SGLang's (Mooncake / NIXL), which this module stands in for.
"""
from __future__ import annotations

import io
import itertools
import json
import struct
from typing import Optional, Sequence

import torch

MAGIC = b"MBKV1\x00"


def pack_blob(blob: Optional[dict]) -> bytes:
    """One binary message: magic, JSON header, raw tensors (``torch.save`` of plain tensors only)."""
    if blob is None:
        return MAGIC + struct.pack("<I", 0)
    head = json.dumps({"tokens": blob["tokens"], "page_size": blob["page_size"], "weight_version": blob["weight_version"]}).encode()
    buf = io.BytesIO()
    torch.save({"kv": blob["kv"].cpu(), "routed_experts": blob.get("routed_experts")}, buf)
    return MAGIC + struct.pack("<I", len(head)) + head + buf.getvalue()


def unpack_blob(data: bytes) -> Optional[dict]:
    if not data.startswith(MAGIC):
        raise ValueError("not a key / value hand-over message")
    (n,) = struct.unpack_from("<I", data, len(MAGIC))
    if n == 0:
        return None
    a = len(MAGIC) + 4
    head = json.loads(data[a:a + n].decode())
    tensors = torch.load(io.BytesIO(data[a + n:]), map_location="cpu", weights_only=True)
    return {**head, "kv": tensors["kv"], "routed_experts": tensors.get("routed_experts")}


class PDPair:
    """A prefill engine and a decode engine of one process (tests, or two engines on GPUs of one trainer process)."""

    def __init__(self, prefill_engine, decode_engine):
        self.prefill, self.decode = prefill_engine, decode_engine
        self.transferred_tokens = 0

    def generate(self, prompts: Sequence[Sequence[int]], params=None, **kw) -> list:
        from .core import SamplingParams

        p = params if isinstance(params, SamplingParams) else SamplingParams.from_dict(params or {})
        only_prefill = SamplingParams.from_dict({"max_new_tokens": 1, "temperature": 0.0, "ignore_eos": True})
        # routing replay needs the routed experts of cached prompt tokens as well: the prefill engine records them so
        # that they travel with the pages
        self.prefill.generate([list(x) for x in prompts], only_prefill, return_routed_experts=bool(kw.get("return_routed_experts")))
        for x in prompts:
            blob = self.prefill.export_prefix(list(x), to_cpu=self.prefill.dev != self.decode.dev)
            self.transferred_tokens += self.decode.import_prefix(blob)
        return self.decode.generate([list(x) for x in prompts], p, **kw)


class PDClient:
    """Requests over HTTP: prefill on one of ``prefill_urls``, hand-over, decode on one of ``decode_urls``. ``transport`` is
    ``async (method, url, json_or_bytes) -> (status, body)`` for tests; by default ``utils.http_utils``."""

    def __init__(self, prefill_urls: Sequence[str], decode_urls: Sequence[str], transport=None):
        self.prefill_urls = [u.rstrip("/") for u in prefill_urls]
        self.decode_urls = [u.rstrip("/") for u in decode_urls]
        if not self.prefill_urls or not self.decode_urls:
            raise ValueError("prefill and decode engines come together")
        self._p, self._d = itertools.cycle(self.prefill_urls), itertools.cycle(self.decode_urls)
        self._transport = transport
        self.transferred_tokens = 0

    async def _call(self, url: str, body, raw: bool = False):
        if self._transport is not None:
            return await self._transport("POST", url, body)
        from ..utils import http_utils

        if isinstance(body, (bytes, bytearray)):
            return await http_utils.post_bytes(url, bytes(body))
        if raw:  # a JSON question with a binary answer
            return await http_utils.post_bytes(url, json.dumps(body).encode(), expect_bytes=True, content_type="application/json")
        return await http_utils.post(url, body)

    async def generate(self, payload: dict) -> dict:
        ids = payload["input_ids"]
        pu, du = next(self._p), next(self._d)
        warm = {"input_ids": ids, "sampling_params": {"max_new_tokens": 1, "temperature": 0.0, "ignore_eos": True},
                "return_logprob": False, "return_routed_experts": bool(payload.get("return_routed_experts"))}
        await self._call(pu + "/generate", warm)
        blob = await self._call(pu + "/export_prefix", {"input_ids": ids}, raw=True)
        got = await self._call(du + "/import_prefix", blob)
        self.transferred_tokens += int((got or {}).get("cached_tokens", 0)) if isinstance(got, dict) else 0
        return await self._call(du + "/generate", payload)
