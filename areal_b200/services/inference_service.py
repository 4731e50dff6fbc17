"""Inference service: a gateway in front of several rollout engines.

* router     – registry of engine workers (their RPC servers), round-robin or least-loaded
               placement with session affinity (multi-turn sessions keep hitting the engine that
               holds their KV prefix);
* data proxy – per-session store of everything generated so far (token ids, logprobs, versions),
               the pause flag that makes new requests wait while weights are being swapped, and
               the export of a finished session as a training trajectory;
* gateway    – public routes: ``/generate``, ``/sessions/*``, ``/pause``, ``/continue``,
               ``/set_version``, ``/workers``.
Reference: areal/experimental/inference_service/{gateway,router,data_proxy,controller}.
"""

from __future__ import annotations

import asyncio
import threading
import time
import uuid
from dataclasses import dataclass, field
from typing import Any

from fastapi import FastAPI, HTTPException, Request

from ..infra.rpc.serialization import deserialize_value, serialize_value
from ..infra.utils.http import request_with_retry
from .base import WorkerRegistry, forward, make_auth


@dataclass
class Session:
    session_id: str
    created: float = field(default_factory=time.time)
    turns: list[dict] = field(default_factory=list)  # one dict per completed generate call
    reward: float | None = None
    finished: bool = False


class SessionStore:
    def __init__(self, ttl: float = 3600.0):
        self.ttl = ttl
        self._s: dict[str, Session] = {}
        self._lock = threading.Lock()

    def start(self, session_id: str | None = None) -> Session:
        with self._lock:
            sid = session_id or uuid.uuid4().hex
            s = self._s[sid] = Session(sid)
            return s

    def get(self, sid: str) -> Session:
        with self._lock:
            s = self._s.get(sid)
        if s is None:
            raise HTTPException(status_code=404, detail=f"unknown session {sid}")
        return s

    def append(self, sid: str, turn: dict):
        self.get(sid).turns.append(turn)

    def finish(self, sid: str, reward: float | None) -> Session:
        s = self.get(sid)
        s.reward, s.finished = reward, True
        return s

    def pop(self, sid: str) -> Session:
        with self._lock:
            s = self._s.pop(sid, None)
        if s is None:
            raise HTTPException(status_code=404, detail=f"unknown session {sid}")
        return s

    def gc(self) -> int:
        now = time.time()
        with self._lock:
            dead = [k for k, s in self._s.items() if now - s.created > self.ttl]
            for k in dead:
                del self._s[k]
        return len(dead)

    def export(self, sid: str) -> dict[str, Any]:
        """A finished session as one trajectory: the last turn's input already contains all earlier
        turns, so the sequence is its input + output; loss covers every generated span."""
        s = self.get(sid)
        if not s.turns:
            raise HTTPException(status_code=409, detail="session has no completed generation")
        seq: list[int] = []
        logp: list[float] = []
        mask: list[int] = []
        ver: list[int] = []
        for t in s.turns:
            new_in = t["input_tokens"][len(seq):]
            seq += new_in + t["output_tokens"]
            logp += [0.0] * len(new_in) + t["output_logprobs"]
            mask += [0] * len(new_in) + [1] * len(t["output_tokens"])
            ver += [-1] * len(new_in) + t["output_versions"]
        return dict(input_ids=seq, logprobs=logp, loss_mask=mask, versions=ver, reward=s.reward)


def create_gateway_app(token: str | None = None, strategy: str = "round_robin", post=None) -> FastAPI:
    app = FastAPI()
    reg = WorkerRegistry(strategy)
    store = SessionStore()
    auth = make_auth(token)
    state = {"paused": False, "version": 0}
    resume = asyncio.Event()
    resume.set()
    post = post or (lambda url, body: request_with_retry("POST", url, json=body, max_retries=0, timeout=3600).json())

    def call_engine(method: str, session_id: str | None, *args, **kwargs):
        payload = {"method": method, "args": serialize_value(list(args)), "kwargs": serialize_value(kwargs)}
        return deserialize_value(forward(reg, "/call", payload, session_id, post=post)["result"])

    @app.post("/register")
    async def register(req: Request):
        auth(req)
        b = await req.json()
        reg.register(b["worker_id"], b["addr"])
        return {"workers": len(reg.snapshot())}

    @app.get("/workers")
    def workers(req: Request):
        auth(req)
        return {"workers": reg.snapshot(), "paused": state["paused"], "version": state["version"]}

    @app.post("/sessions/start")
    async def start(req: Request):
        auth(req)
        b = await req.json() if await req.body() else {}
        return {"session_id": store.start(b.get("session_id")).session_id}

    @app.post("/generate")
    async def generate(req: Request):
        auth(req)
        b = await req.json()
        while state["paused"]:  # weights are being swapped: hold the request, do not fail it
            resume.clear()
            await asyncio.wait_for(resume.wait(), timeout=3600)
        sid = b.get("session_id")
        model_req = deserialize_value(b["request"])
        resp = await asyncio.get_running_loop().run_in_executor(None, lambda: call_engine("generate", sid, model_req))
        turn = dict(input_tokens=list(resp.input_tokens), output_tokens=list(resp.output_tokens),
                    output_logprobs=list(resp.output_logprobs), output_versions=list(resp.output_versions),
                    stop_reason=resp.stop_reason)
        if sid is not None:
            store.append(sid, turn)
        return {"response": serialize_value(resp)}

    @app.post("/sessions/{sid}/finish")
    async def finish(sid: str, req: Request):
        auth(req)
        b = await req.json() if await req.body() else {}
        store.finish(sid, b.get("reward"))
        traj = store.export(sid)
        store.pop(sid)
        reg.end_session(sid)
        return {"trajectory": traj}

    @app.post("/pause")
    async def pause(req: Request):
        auth(req)
        state["paused"] = True
        for w in reg.snapshot():
            post(f"http://{w['addr']}/call", {"method": "pause_generation", "args": serialize_value([]),
                                              "kwargs": serialize_value({})})
        return {"paused": True}

    @app.post("/continue")
    async def cont(req: Request):
        auth(req)
        for w in reg.snapshot():
            post(f"http://{w['addr']}/call", {"method": "continue_generation", "args": serialize_value([]),
                                              "kwargs": serialize_value({})})
        state["paused"] = False
        resume.set()
        return {"paused": False}

    @app.post("/set_version")
    async def set_version(req: Request):
        auth(req)
        v = int((await req.json())["version"])
        state["version"] = v
        for w in reg.snapshot():
            post(f"http://{w['addr']}/call", {"method": "set_version", "args": serialize_value([v]),
                                              "kwargs": serialize_value({})})
        return {"version": v}

    app.state.registry, app.state.sessions, app.state.flags = reg, store, state
    return app
