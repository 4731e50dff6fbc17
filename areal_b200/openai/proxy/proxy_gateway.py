"""Session-key gateway in front of several proxy rollout servers.

One public address for external agent programs (anything that speaks the OpenAI or Anthropic API). The
gateway holds no trajectories, only routing state:

* a proxy worker that is ready for an external episode announces itself with
  ``POST /internal/wait_for_session`` (``OnlineAgent`` does this from inside the rollout workflow) and the call
  stays open until that episode is over;
* an external user opens an episode with ``POST /rl/start_session`` (admin key): the gateway takes the oldest
  ready worker, opens a session on it and remembers ``session api key -> worker``;
* ``/v1/chat/completions``, ``/v1/responses``, ``/v1/messages`` and ``/rl/set_reward`` are forwarded to the
  worker that owns the bearer key; ``/rl/end_session`` is forwarded too and then resolves the worker's pending
  ``wait_for_session`` call with the session's id and key, so the workflow on that worker exports the trajectory.

Role of areal/experimental/openai/proxy/proxy_gateway.py (stateless FastAPI gateway with session-pinned
backends and a coordination queue for online training).
"""

from __future__ import annotations

import asyncio
import hmac
from collections import OrderedDict, deque
from dataclasses import dataclass
from typing import Awaitable, Callable

from fastapi import FastAPI, HTTPException, Request, Response

FORWARDED = ("/v1/chat/completions", "/v1/responses", "/v1/messages", "/rl/set_reward")

# (method, url, json body, headers) -> (status, body bytes, content type)
Forwarder = Callable[[str, str, dict, dict], Awaitable[tuple[int, bytes, str]]]


@dataclass
class _Ready:
    worker_addr: str
    future: asyncio.Future  # resolves to {"session_id", "api_key"} when the episode has ended


async def _aiohttp_forward(method: str, url: str, body: dict, headers: dict) -> tuple[int, bytes, str]:
    import aiohttp

    async with aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=3600)) as s:
        async with s.request(method, url, json=body, headers=headers) as r:
            return r.status, await r.read(), r.headers.get("content-type", "application/json")


def create_gateway_app(admin_api_key: str = "areal-admin-key", forward: Forwarder | None = None,
                       max_routes: int = 100_000) -> FastAPI:
    """``forward`` performs the backend HTTP call (default: aiohttp); tests pass an in-process one."""
    app = FastAPI()
    fwd = forward or _aiohttp_forward
    ready: deque[_Ready] = deque()
    routes: "OrderedDict[str, tuple[str, str, asyncio.Future]]" = OrderedDict()  # session key -> (worker, session id, future)
    arrival = asyncio.Condition()

    def bearer(req: Request) -> str:
        auth = req.headers.get("authorization") or req.headers.get("x-api-key") or ""
        return auth[7:] if auth.lower().startswith("bearer ") else auth

    def require_admin(req: Request):
        if not hmac.compare_digest(bearer(req), admin_api_key):
            raise HTTPException(status_code=401, detail="admin key required")

    def _url(worker: str, path: str) -> str:
        return (worker if worker.startswith("http") else "http://" + worker).rstrip("/") + path

    @app.get("/health")
    def health():
        return {"status": "ok", "ready_workers": len(ready), "sessions": len(routes)}

    @app.post("/internal/wait_for_session")
    async def wait_for_session(req: Request):
        require_admin(req)
        b = await req.json()
        entry = _Ready(b["worker_addr"], asyncio.get_running_loop().create_future())
        ready.append(entry)
        async with arrival:
            arrival.notify_all()
        try:
            info = await asyncio.wait_for(entry.future, timeout=float(b.get("timeout", 3600.0)))
        except asyncio.TimeoutError:
            if entry in ready:
                ready.remove(entry)
            raise HTTPException(status_code=408, detail="no external session arrived in time")
        return info

    @app.post("/rl/start_session")
    async def start_session(req: Request):
        require_admin(req)
        body = await req.json() if await req.body() else {}
        wait_s = float(body.pop("wait_for_worker", 0.0) or 0.0)
        if not ready and wait_s > 0:
            async with arrival:
                try:
                    await asyncio.wait_for(arrival.wait_for(lambda: bool(ready)), timeout=wait_s)
                except asyncio.TimeoutError:
                    pass
        if not ready:
            raise HTTPException(status_code=503, detail="no proxy worker is waiting for an external session")
        entry = ready.popleft()
        status, raw, ctype = await fwd("POST", _url(entry.worker_addr, "/rl/start_session"), body,
                                       {"Authorization": f"Bearer {admin_api_key}"})
        if status != 200:
            ready.appendleft(entry)
            return Response(content=raw, status_code=status, media_type=ctype)
        import json

        sess = json.loads(raw)
        routes[sess["api_key"]] = (entry.worker_addr, sess["session_id"], entry.future)
        while len(routes) > max_routes:
            routes.popitem(last=False)
        return sess

    async def _route(req: Request, path: str):
        key = bearer(req)
        r = routes.get(key)
        if r is None:
            raise HTTPException(status_code=401, detail="unknown session key")
        body = await req.json() if await req.body() else {}
        status, raw, ctype = await fwd("POST", _url(r[0], path), body, {"Authorization": f"Bearer {key}"})
        return key, r, Response(content=raw, status_code=status, media_type=ctype)

    def _make(path: str):
        async def handler(req: Request):
            return (await _route(req, path))[2]

        return handler

    for _p in FORWARDED:
        app.post(_p)(_make(_p))

    @app.post("/rl/end_session")
    async def end_session(req: Request):
        key, (worker, sid, fut), resp = await _route(req, "/rl/end_session")
        if resp.status_code == 200:
            routes.pop(key, None)
            if not fut.done():
                fut.set_result({"session_id": sid, "api_key": key, "worker_addr": worker})
        return resp

    app.state.ready, app.state.routes = ready, routes
    return app


create_proxy_gateway_app = create_gateway_app  # the name of the reference's factory
