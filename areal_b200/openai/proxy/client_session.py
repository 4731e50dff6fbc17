"""Client side of one proxy session.

``async with OpenAIProxyClient(proxy_url, admin_api_key) as s:`` opens a session on a proxy rollout server (or
on the gateway in front of several), hands out what an agent needs to talk to the model (``s.base_url``,
``s.session_api_key``: any OpenAI-compatible SDK takes them) and ends the session on exit. Rewards go to single
completions (``set_reward``) or to the last one (``set_last_reward``); ``export_interactions`` returns the
recorded completions as training tensors (token ids, log-probs, loss mask, weight versions, rewards propagated
backwards with ``discount``). ``post`` is injectable (tests, other HTTP stacks); the default uses aiohttp with a
few retries on connection errors and 5xx answers.

Reference: areal/experimental/openai/proxy/client_session.py (OpenAIProxyClient :39, set_interaction_reward
:308, set_last_interaction_reward :324).
"""

from __future__ import annotations

import asyncio
from typing import Any, Awaitable, Callable

Post = Callable[[str, dict, dict], Awaitable[dict]]


class ProxyRequestError(RuntimeError):
    def __init__(self, url: str, status: int | None, body: str):
        self.url, self.status, self.body = url, status, body
        super().__init__(f"POST {url} failed ({status}): {body[:300]}")


def should_retry(exc: BaseException) -> bool:
    """Connection trouble and server-side errors are retried; a 4xx answer is the caller's mistake."""
    if isinstance(exc, ProxyRequestError):
        return exc.status is None or exc.status >= 500
    return isinstance(exc, (ConnectionError, asyncio.TimeoutError, OSError))


async def post_json(url: str, body: dict, headers: dict, timeout: float = 600.0) -> dict:
    import aiohttp

    try:
        async with aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=timeout)) as s:
            async with s.post(url, json=body, headers=headers) as r:
                text = await r.text()
                if r.status >= 400:
                    raise ProxyRequestError(url, r.status, text)
                return await r.json(content_type=None) if text else {}
    except aiohttp.ClientConnectionError as e:
        raise ProxyRequestError(url, None, str(e)) from e


async def post_json_with_retry(url: str, body: dict, headers: dict, post: Post | None = None, retries: int = 3,
                               delay: float = 0.5) -> dict:
    post = post or post_json
    for attempt in range(retries + 1):
        try:
            return await post(url, body, headers)
        except BaseException as e:  # noqa: BLE001 - filtered by should_retry
            if attempt == retries or not should_retry(e):
                raise
            await asyncio.sleep(delay * (2 ** attempt))
    raise AssertionError("unreachable")


async def set_interaction_reward(base_url: str, api_key: str, interaction_id: str, reward: float,
                                 post: Post | None = None) -> dict:
    """Reward of one recorded completion of the session that ``api_key`` belongs to."""
    return await post_json_with_retry(f"{base_url.rstrip('/')}/rl/set_reward",
                                      {"interaction_id": interaction_id, "reward": float(reward)},
                                      {"Authorization": f"Bearer {api_key}"}, post)


async def set_last_interaction_reward(base_url: str, api_key: str, reward: float, post: Post | None = None) -> dict:
    return await post_json_with_retry(f"{base_url.rstrip('/')}/rl/set_reward", {"reward": float(reward)},
                                      {"Authorization": f"Bearer {api_key}"}, post)


class OpenAIProxyClient:
    def __init__(self, proxy_url: str, admin_api_key: str = "areal-admin-key", task_id: str | None = None,
                 post: Post | None = None, retries: int = 3):
        self.proxy_url = proxy_url.rstrip("/")
        self.admin_api_key, self.task_id = admin_api_key, task_id
        self._post, self.retries = post, retries
        self.session_id: str | None = None
        self._key: str | None = None
        self._ended = False

    # what the agent needs
    @property
    def base_url(self) -> str:
        return f"{self.proxy_url}/v1"

    @property
    def session_api_key(self) -> str:
        if self._key is None:
            raise RuntimeError("the session has not been started (use `async with`)")
        return self._key

    def _admin(self) -> dict[str, str]:
        return {"Authorization": f"Bearer {self.admin_api_key}"}

    def _session(self) -> dict[str, str]:
        return {"Authorization": f"Bearer {self.session_api_key}"}

    async def _call(self, path: str, body: dict, headers: dict) -> dict:
        return await post_json_with_retry(self.proxy_url + path, body, headers, self._post, self.retries)

    # lifecycle
    async def start(self) -> "OpenAIProxyClient":
        out = await self._call("/rl/start_session", {"task_id": self.task_id} if self.task_id else {}, self._admin())
        self.session_id, self._key = out["session_id"], out["api_key"]
        return self

    async def end(self) -> None:
        if self._key is not None and not self._ended:
            self._ended = True
            await self._call("/rl/end_session", {}, self._session())

    async def __aenter__(self) -> "OpenAIProxyClient":
        return await self.start()

    async def __aexit__(self, exc_type, exc, tb) -> None:
        try:
            await self.end()
        except Exception:  # noqa: BLE001 - do not hide the body's exception behind a failed clean-up
            if exc_type is None:
                raise

    # rewards and export
    async def set_reward(self, completion_id: str, reward: float) -> dict:
        return await self._call("/rl/set_reward", {"interaction_id": completion_id, "reward": float(reward)},
                                self._session())

    async def set_last_reward(self, reward: float) -> dict:
        return await self._call("/rl/set_reward", {"reward": float(reward)}, self._session())

    async def export_interactions(self, discount: float = 1.0, style: str = "individual") -> dict[str, Any]:
        """``{completion id: tensor dict}`` of the session (ends it first if it is still open)."""
        from ...infra.rpc.serialization import deserialize_value

        await self.end()
        out = await self._call("/export_trajectories",
                               {"session_id": self.session_id, "discount": discount, "style": style}, self._admin())
        return {k: deserialize_value(v) for k, v in out["interactions"].items()}
