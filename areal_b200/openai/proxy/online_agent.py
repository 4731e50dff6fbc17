"""Agent of ``online`` mode: the real agent is an external program that reaches the proxy through the gateway.
``run`` announces this worker to the gateway as ready for one external episode and returns when that episode
is over, with the credentials of the session the external user held, so that the workflow exports the
session's trajectory from the local proxy server (role of areal/experimental/openai/proxy/online_agent.py).
Without a gateway address it only waits ``wait_seconds`` (an external agent that was given ``base_url`` /
``api_key`` directly reports through ``POST /rl/set_reward``)."""

from __future__ import annotations

import asyncio
from typing import Any


class OnlineAgent:
    def __init__(self, gateway_url: str | None = None, worker_addr: str | None = None,
                 admin_api_key: str = "areal-admin-key", timeout: float = 3600.0, wait_seconds: float = 0.0,
                 post=None):
        """``post(url, json, headers) -> dict``: the HTTP call (default: aiohttp); tests inject an in-process one."""
        self.gateway_url, self.worker_addr = gateway_url, worker_addr
        self.admin_api_key, self.timeout, self.wait_seconds = admin_api_key, timeout, wait_seconds
        self._post = post

    async def _http_post(self, url: str, body: dict, headers: dict) -> dict:
        if self._post is not None:
            return await self._post(url, body, headers)
        import aiohttp

        async with aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=self.timeout + 30)) as s:
            async with s.post(url, json=body, headers=headers) as r:
                r.raise_for_status()
                return await r.json()

    async def run(self, data: dict[str, Any], **extra: Any):
        if not self.gateway_url:
            if self.wait_seconds:
                await asyncio.sleep(self.wait_seconds)
            return None
        info = await self._http_post(f"{self.gateway_url.rstrip('/')}/internal/wait_for_session",
                                     {"worker_addr": self.worker_addr, "timeout": self.timeout},
                                     {"Authorization": f"Bearer {self.admin_api_key}"})
        return info  # {"session_id", "api_key", "worker_addr"} of the finished external session
