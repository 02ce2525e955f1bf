"""Shared async HTTP client with bounded retries (rollout functions, remote reward models, router registration).

Reference: miles/utils/http_utils.py (368 lines: shared httpx client, post/get with retries).
"""
from __future__ import annotations

import asyncio
import random
from typing import Any, Optional

_client = None
_limits = {"max_connections": 1024, "timeout": 600.0}


def configure(max_connections: int = 1024, timeout: float = 600.0) -> None:
    global _client
    _limits.update(max_connections=max_connections, timeout=timeout)
    _client = None


_client_loop = None


def client():
    """The shared client of the running event loop (connections belong to a loop: a client made under an earlier
    ``asyncio.run`` is replaced, not reused)."""
    global _client, _client_loop
    try:
        loop = asyncio.get_running_loop()
    except RuntimeError:
        loop = None
    if _client is None or _client_loop is not loop:
        import httpx

        _client = httpx.AsyncClient(timeout=_limits["timeout"], limits=httpx.Limits(max_connections=_limits["max_connections"]))
        _client_loop = loop
    return _client


async def request(method: str, url: str, payload: Optional[dict] = None, max_retries: int = 5, base_delay: float = 0.5,
                  retry_on=(500, 502, 503, 504), transport=None) -> Any:
    """JSON request with exponential back-off and jitter. ``transport(method, url, payload) -> (status, json)`` replaces
    the network in tests. Raises the last error when every attempt failed."""
    last: Optional[BaseException] = None
    for attempt in range(max_retries + 1):
        try:
            if transport is not None:
                status, body = await transport(method, url, payload)
            else:
                r = await client().request(method, url, json=payload)
                status, body = r.status_code, (r.json() if r.content else None)
            if status in retry_on:
                raise RuntimeError(f"{method} {url} -> HTTP {status}")
            if status >= 400:
                raise ValueError(f"{method} {url} -> HTTP {status}: {body}")
            return body
        except ValueError:
            raise  # the request itself is wrong: retrying cannot help
        except Exception as e:  # noqa: BLE001 - network errors of any kind are retried
            last = e
            if attempt == max_retries:
                break
            await asyncio.sleep(base_delay * (2 ** attempt) * (0.5 + random.random() / 2))
    raise last if last is not None else RuntimeError("request failed")


async def post(url: str, payload: Optional[dict] = None, **kw) -> Any:
    return await request("POST", url, payload, **kw)


async def get(url: str, **kw) -> Any:
    return await request("GET", url, None, **kw)


async def post_bytes(url: str, body: bytes, expect_bytes: bool = False, content_type: str = "application/octet-stream",
                     max_retries: int = 3, base_delay: float = 0.5) -> Any:
    """POST a raw body (binary hand-over messages); returns the raw response body, or its JSON when ``expect_bytes`` is
    false. A JSON request that expects a binary answer passes ``content_type="application/json"``."""
    last: Optional[BaseException] = None
    for attempt in range(max_retries + 1):
        try:
            r = await client().post(url, content=body, headers={"content-type": content_type})
            if r.status_code >= 500:
                raise RuntimeError(f"POST {url} -> HTTP {r.status_code}")
            if r.status_code >= 400:
                raise ValueError(f"POST {url} -> HTTP {r.status_code}: {r.text[:200]}")
            return r.content if expect_bytes else (r.json() if r.content else None)
        except ValueError:
            raise
        except Exception as e:  # noqa: BLE001
            last = e
            if attempt == max_retries:
                break
            await asyncio.sleep(base_delay * (2 ** attempt) * (0.5 + random.random() / 2))
    raise last if last is not None else RuntimeError("request failed")
