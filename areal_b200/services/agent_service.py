"""Agent service: runs user "agent runnables" (any object with ``async run(data, **kw)`` that
talks to an OpenAI-compatible ``base_url``) on worker processes, one session per episode.

* worker  – ``/run`` instantiates the runnable (import path + kwargs), gives it the session's
            ``base_url`` / ``api_key`` and returns its reward;
* gateway – ``/sessions/start`` picks a worker (least loaded), ``/sessions/{id}/run`` forwards
            with session affinity, ``/sessions/{id}/end`` releases the session. With ``agent=`` it also serves
            ``/v1/responses`` (the OpenAI Responses protocol): ``user`` names the conversation, the gateway keeps
            its history (the data-proxy role) and hands ``{"input", "history"}`` to the agent on the session's
            worker; the agent's text comes back as a ``response`` object.
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


def _input_messages(inp) -> list[dict]:
    """The ``input`` of a Responses request as chat messages: a string, or items ``{"type": "message", "role",
    "content"}`` whose content is a string or a list of ``input_text`` parts."""
    if isinstance(inp, str):
        return [{"role": "user", "content": inp}]
    out = []
    for item in inp or []:
        if isinstance(item, str):
            out.append({"role": "user", "content": item})
            continue
        if item.get("type", "message") != "message":
            continue
        c = item.get("content", "")
        if isinstance(c, list):
            c = "".join(part.get("text", "") for part in c if isinstance(part, dict))
        out.append({"role": item.get("role", "user"), "content": c})
    return out


def create_gateway_app(token: str | None = None, post=None, agent: str | None = None,
                       agent_kwargs: dict | None = None, base_url: str | None = None,
                       api_key: str | None = None, max_history: int = 64) -> FastAPI:
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

    conversations: dict[str, list[dict]] = {}

    @app.post("/v1/responses")
    async def responses(req: Request):
        auth(req)
        if agent is None:
            raise HTTPException(status_code=501, detail="this gateway was started without an agent")
        b = await req.json()
        user = str(b.get("user") or uuid.uuid4().hex)
        new = _input_messages(b.get("input"))
        if not new:
            raise HTTPException(status_code=400, detail="`input` holds no message")
        history = conversations.setdefault(user, [])
        if user not in sessions:
            sessions[user] = {"base_url": base_url, "api_key": api_key, "runs": 0}
            reg.pick(user)
        sessions[user]["runs"] += 1
        payload = {"agent": agent, "agent_kwargs": serialize_value(agent_kwargs or {}),
                   "data": serialize_value({"input": new, "history": list(history), "model": b.get("model")}),
                   "base_url": base_url, "api_key": api_key}
        out = deserialize_value(forward(reg, "/run", payload, user, post=post)["result"])
        text = out.get("output_text", "") if isinstance(out, dict) else str(out)
        history.extend(new)
        history.append({"role": "assistant", "content": text})
        del history[:-max_history]
        rid = "resp_" + uuid.uuid4().hex
        return {"id": rid, "object": "response", "status": "completed", "model": b.get("model") or "agent",
                "user": user, "output_text": text,
                "output": [{"type": "message", "id": "msg_" + rid[5:], "role": "assistant", "status": "completed",
                            "content": [{"type": "output_text", "text": text, "annotations": []}]}],
                "metadata": {k: v for k, v in out.items() if k != "output_text"} if isinstance(out, dict) else {}}

    @app.post("/v1/conversations/{user}/reset")
    async def reset(user: str, req: Request):
        auth(req)
        n = len(conversations.pop(user, []))
        if sessions.pop(user, None) is not None:
            reg.end_session(user)
        return {"dropped_messages": n}

    app.state.registry = reg
    app.state.conversations = conversations
    return app
