"""Agent service: runs user "agent runnables" (any object with ``async run(data, **kw)`` that
talks to an OpenAI-compatible ``base_url``) on worker processes, one session per episode.

* worker  – ``/run`` instantiates the runnable (import path + kwargs), gives it the session's
            ``base_url`` / ``api_key`` and returns its reward;
* gateway – ``/sessions/start`` picks a worker (least loaded), ``/sessions/{id}/run`` forwards
            with session affinity, ``/sessions/{id}/end`` releases the session.
Reference: areal/experimental/agent_service/{gateway,router,data_proxy,worker}, protocol.py.
"""

from __future__ import annotations

import importlib
import inspect
import uuid

from fastapi import FastAPI, HTTPException, Request

from ..infra.rpc.serialization import deserialize_value, serialize_value
from ..infra.utils.http import request_with_retry
from .base import WorkerRegistry, forward, make_auth


def create_worker_app() -> FastAPI:
    app = FastAPI()
    cache: dict[str, object] = {}

    @app.get("/health")
    def health():
        return {"status": "ok"}

    @app.post("/run")
    async def run(req: Request):
        b = await req.json()
        path, kwargs = b["agent"], deserialize_value(b.get("agent_kwargs", {}))
        key = path + repr(sorted(kwargs.items()))
        agent = cache.get(key)
        if agent is None:
            mod, _, attr = path.rpartition(".")
            try:
                obj = getattr(importlib.import_module(mod), attr)
            except (ImportError, AttributeError) as e:
                raise HTTPException(status_code=400, detail=f"cannot import agent {path!r}: {e}")
            agent = cache[key] = obj(**kwargs) if inspect.isclass(obj) else obj
        fn = agent.run if hasattr(agent, "run") else agent
        extra = {"base_url": b.get("base_url"), "api_key": b.get("api_key")}
        accepted = inspect.signature(fn).parameters
        if not any(p.kind == p.VAR_KEYWORD for p in accepted.values()):
            extra = {k: v for k, v in extra.items() if k in accepted}
        out = fn(deserialize_value(b.get("data", {})), **extra)
        if inspect.isawaitable(out):
            out = await out
        return {"result": serialize_value(out)}

    return app


def create_gateway_app(token: str | None = None, post=None) -> FastAPI:
    app = FastAPI()
    reg = WorkerRegistry("least_loaded")
    auth = make_auth(token)
    post = post or (lambda url, body: request_with_retry("POST", url, json=body, max_retries=0, timeout=7200).json())
    sessions: dict[str, dict] = {}

    @app.post("/register")
    async def register(req: Request):
        auth(req)
        b = await req.json()
        reg.register(b["worker_id"], b["addr"])
        return {"workers": len(reg.snapshot())}

    @app.post("/sessions/start")
    async def start(req: Request):
        auth(req)
        b = await req.json() if await req.body() else {}
        sid = uuid.uuid4().hex
        sessions[sid] = {"base_url": b.get("base_url"), "api_key": b.get("api_key"), "runs": 0}
        reg.pick(sid)  # binds the session to a worker
        return {"session_id": sid}

    @app.post("/sessions/{sid}/run")
    async def run(sid: str, req: Request):
        auth(req)
        if sid not in sessions:
            raise HTTPException(status_code=404, detail=f"unknown session {sid}")
        b = await req.json()
        payload = dict(b, base_url=sessions[sid]["base_url"], api_key=sessions[sid]["api_key"])
        sessions[sid]["runs"] += 1
        return forward(reg, "/run", payload, sid, post=post)

    @app.post("/sessions/{sid}/end")
    async def end(sid: str, req: Request):
        auth(req)
        info = sessions.pop(sid, None)
        if info is None:
            raise HTTPException(status_code=404, detail=f"unknown session {sid}")
        reg.end_session(sid)
        return {"runs": info["runs"]}

    app.state.registry = reg
    return app
