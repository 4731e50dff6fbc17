"""Placeholder agent of ``online`` mode: the real agent is an external program that calls the
proxy with the session's ``base_url`` / ``api_key``; this object only waits for it to finish
(role of areal/experimental/openai/proxy/online_agent.py)."""

from __future__ import annotations

import asyncio
from typing import Any


class OnlineAgent:
    def __init__(self, wait_seconds: float = 0.0):
        self.wait_seconds = wait_seconds

    async def run(self, data: dict[str, Any], **extra: Any):
        # the external agent reports its reward through POST /rl/set_reward
        if self.wait_seconds:
            await asyncio.sleep(self.wait_seconds)
        return None
