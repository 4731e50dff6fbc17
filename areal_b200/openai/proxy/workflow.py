"""Runs an agent (any object with ``async run(data, **extra)``) as a rollout workflow.

* ``inline``  – the agent runs inside the rollout process and receives an
  :class:`ArealOpenAI` client (``extra["client"]``) bound to the engine;
* ``subproc`` – the agent coroutine runs in a worker thread with its own event
  loop (for agents that block), same client;
* ``online``  – the agent is an external program: the workflow opens an RL
  session on the proxy server, hands ``base_url`` / ``api_key`` to the agent
  and exports the session's trajectories when the agent is done.

The agent's return value is the reward: a float for the last interaction or a
``{interaction_id: reward}`` mapping (role of
areal/experimental/openai/proxy/workflow.py:72).
"""

from __future__ import annotations

import asyncio
from concurrent.futures import ThreadPoolExecutor
from typing import Any

from ...api.cli_args import GenerationHyperparameters
from ...api.workflow_api import RolloutWorkflow
from ..client import ArealOpenAI


class OpenAIProxyWorkflow(RolloutWorkflow):
    def __init__(self, agent: Any, tokenizer=None, gconfig: GenerationHyperparameters | None = None,
                 mode: str = "inline", turn_discount: float = 1.0, export_style: str = "individual",
                 proxy_url: str | None = None, admin_api_key: str = "areal-admin-key",
                 tool_call_parser: str = "qwen", reasoning_parser: str | None = None, max_workers: int = 4,
                 processor=None):
        self.processor = processor  # vision-language models: expands image_url message parts
        if mode not in ("inline", "subproc", "online"):
            raise ValueError(f"mode must be inline|subproc|online, got {mode}")
        self.agent, self.tokenizer, self.gconfig, self.mode = agent, tokenizer, gconfig, mode
        self.turn_discount, self.export_style = turn_discount, export_style
        self.proxy_url, self.admin_api_key = proxy_url, admin_api_key
        self.tool_call_parser, self.reasoning_parser = tool_call_parser, reasoning_parser
        self._pool = ThreadPoolExecutor(max_workers) if mode == "subproc" else None

    async def arun_episode(self, engine, data: dict[str, Any]):
        if self.mode == "online":
            return await self._run_online(data)
        client = ArealOpenAI(engine, self.tokenizer, self.gconfig, self.tool_call_parser, self.reasoning_parser,
                             processor=self.processor)
        if self.mode == "inline":
            reward = await self.agent.run(data, client=client)
        else:
            loop = asyncio.get_running_loop()
            main_loop = loop

            class _Bridge:
                """Lets the worker thread's coroutine call the engine on the main loop."""

                def __init__(self, c):
                    self._c = c
                    self.chat = type("chat", (), {"completions": self})()

                async def create(self, **kw):
                    fut = asyncio.run_coroutine_threadsafe(self._c.chat.completions.create(**kw), main_loop)
                    return await asyncio.wrap_future(fut)

            bridge = _Bridge(client)
            reward = await loop.run_in_executor(self._pool, lambda: asyncio.run(self.agent.run(data, client=bridge)))
        if not client.cache:
            return None
        if isinstance(reward, dict):
            for k, v in reward.items():
                client.set_reward(k, float(v))
        elif reward is not None:
            client.set_last_reward(float(reward))
        return client.export_interactions(self.export_style, self.turn_discount)

    async def _run_online(self, data):
        from ...utils.data import concat_padded_tensors
        from .client_session import OpenAIProxyClient

        assert self.proxy_url, "online mode needs proxy_url"
        async with OpenAIProxyClient(self.proxy_url, self.admin_api_key) as sess:
            reward = await self.agent.run(data, base_url=sess.base_url, api_key=sess.session_api_key)
            if isinstance(reward, dict) and "session_id" in reward and "api_key" in reward:
                # an online agent that waited at the gateway: the external user's session is the one to export
                await sess.end()  # the workflow's own (unused) session
                sess.session_id, sess._key = reward["session_id"], reward["api_key"]
            elif isinstance(reward, dict):
                for k, v in reward.items():
                    await sess.set_reward(k, v)
            elif reward is not None:
                await sess.set_last_reward(float(reward))
            inter = await sess.export_interactions(self.turn_discount, self.export_style)
        if not inter:
            return None
        return concat_padded_tensors(list(inter.values()))
