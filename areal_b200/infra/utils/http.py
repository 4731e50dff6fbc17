"""HTTP helpers with retries and exponential back-off (areal/infra/utils/http.py in the reference,
which uses tenacity)."""

from __future__ import annotations

import asyncio
import time
from typing import Any

import requests


class HTTPRequestError(RuntimeError):
    def __init__(self, url: str, status: int | None, detail: str):
        super().__init__(f"{url}: HTTP {status}: {detail}")
        self.url, self.status, self.detail = url, status, detail


def request_with_retry(method: str, url: str, *, json: Any = None, timeout: float = 30.0, max_retries: int = 3,
                       backoff: float = 0.5, retry_statuses=(502, 503, 504),
                       headers: dict[str, str] | None = None) -> requests.Response:
    last: Exception | None = None
    for attempt in range(max_retries + 1):
        try:
            r = requests.request(method, url, json=json, timeout=timeout, headers=headers or None)
            if r.status_code in retry_statuses and attempt < max_retries:
                last = HTTPRequestError(url, r.status_code, r.text[:200])
            else:
                if r.status_code >= 400:
                    raise HTTPRequestError(url, r.status_code, r.text[:500])
                return r
        except (requests.ConnectionError, requests.Timeout) as e:
            last = e
            if attempt == max_retries:
                break
        time.sleep(backoff * (2 ** attempt))
    raise HTTPRequestError(url, None, f"gave up after {max_retries + 1} attempts: {last}")


async def arequest_with_retry(session, method: str, url: str, *, json: Any = None, timeout: float = 30.0,
                              max_retries: int = 3, backoff: float = 0.5, retry_statuses=(502, 503, 504),
                              headers: dict[str, str] | None = None) -> Any:
    """aiohttp variant; returns the decoded JSON body."""
    import aiohttp

    last: Exception | None = None
    for attempt in range(max_retries + 1):
        try:
            async with session.request(method, url, json=json, headers=headers or None,
                                       timeout=aiohttp.ClientTimeout(total=timeout)) as r:
                if r.status in retry_statuses and attempt < max_retries:
                    last = HTTPRequestError(url, r.status, (await r.text())[:200])
                else:
                    if r.status >= 400:
                        raise HTTPRequestError(url, r.status, (await r.text())[:500])
                    return await r.json()
        except (aiohttp.ClientConnectionError, asyncio.TimeoutError) as e:
            last = e
            if attempt == max_retries:
                break
        await asyncio.sleep(backoff * (2 ** attempt))
    raise HTTPRequestError(url, None, f"gave up after {max_retries + 1} attempts: {last}")
