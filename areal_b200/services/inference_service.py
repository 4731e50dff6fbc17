"""Inference service: a gateway in front of several rollout engines.

* router     – registry of engine workers (their RPC servers), round-robin or least-loaded
               placement with session affinity (multi-turn sessions keep hitting the engine that
               holds their KV prefix);
* data proxy – per-session store of everything generated so far (token ids, logprobs, versions),
               the pause flag that makes new requests wait while weights are being swapped, and
               the export of a finished session as a training trajectory;
* gateway    – public routes: ``/generate``, ``/sessions/*``, ``/pause``, ``/continue``,
               ``/set_version``, ``/workers``; with a tokenizer also ``/v1/chat/completions`` (OpenAI
               protocol over the engines, recorded per session and exported as training tensors by
               ``/sessions/{id}/export_chat``) with *external models*: chat requests that name a
               configured external model are forwarded to that provider instead.
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


def create_gateway_app(token: str | None = None, strategy: str = "round_robin", post=None, tokenizer=None,
                       external_models: dict[str, dict] | None = None, external_post=None) -> FastAPI:
    """``tokenizer``: turns on ``POST /v1/chat/completions`` (OpenAI protocol; ``session_id`` in the body or an
    ``X-Session-Id`` header keeps a conversation on one engine and records it for export).
    ``external_models``: ``{model name: {"url": ..., "api_key": ...}}``: chat requests that name such a model
    are forwarded to that OpenAI-compatible endpoint instead of the engines (a user simulator or a judge that
    is not the policy); they are not recorded. ``external_post(url, body, headers) -> dict`` is its transport."""
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

    external = dict(external_models or {})
    external_post = external_post or (lambda url, body, headers: request_with_retry(
        "POST", url, json=body, headers=headers, max_retries=2, timeout=600).json())
    chat_clients: dict[str, Any] = {}  # session id -> the OpenAI-protocol client that records its completions

    class _RoutedEngine:
        """What the protocol client sees as its engine: generation goes through the registry, pinned to a session."""

        def __init__(self, sid):
            self.sid = sid

        async def agenerate(self, req):
            while state["paused"]:
                resume.clear()
                await asyncio.wait_for(resume.wait(), timeout=3600)
            import dataclasses

            wire = dataclasses.replace(req, tokenizer=None)  # the engine worker has its own; it does not travel
            resp = await asyncio.get_running_loop().run_in_executor(None, lambda: call_engine("generate", self.sid, wire))
            resp.tokenizer = req.tokenizer
            return resp

        def get_version(self):
            return state["version"]

    @app.post("/v1/chat/completions")
    async def chat_completions(req: Request):
        auth(req)
        b = await req.json()
        model = b.get("model", "default")
        if model in external:
            ext = external[model]
            body = {k: v for k, v in b.items() if k != "session_id"}
            body["model"] = ext.get("model", model)
            headers = {"Authorization": f"Bearer {ext['api_key']}"} if ext.get("api_key") else {}
            return await asyncio.get_running_loop().run_in_executor(
                None, lambda: external_post(ext["url"].rstrip("/") + "/chat/completions", body, headers))
        if tokenizer is None:
            raise HTTPException(status_code=501, detail="this gateway was started without a tokenizer")
        from ..openai.client import ArealOpenAI

        sid = b.get("session_id") or req.headers.get("x-session-id")
        client = chat_clients.get(sid) if sid else None
        if client is None:
            client = ArealOpenAI(_RoutedEngine(sid), tokenizer)
            if sid:
                store.get(sid)  # 404 for a session that was never started
                chat_clients[sid] = client
        return await client._complete(b["messages"], model=model, tools=b.get("tools"),
                                      max_new=b.get("max_completion_tokens") or b.get("max_tokens"),
                                      temperature=b.get("temperature"), top_p=b.get("top_p"), stop=b.get("stop"),
                                      as_dict=True)

    @app.post("/sessions/{sid}/export_chat")
    async def export_chat(sid: str, req: Request):
        """Ends a chat session: rewards the last completion (``reward``) or single ones (``rewards``: id → value)
        and returns the recorded completions as training tensors."""
        auth(req)
        b = await req.json() if await req.body() else {}
        client = chat_clients.pop(sid, None)
        if client is None:
            raise HTTPException(status_code=404, detail=f"session {sid} has no chat completions")
        for k, v in (b.get("rewards") or {}).items():
            client.set_reward(k, float(v))
        if b.get("reward") is not None:
            client.set_last_reward(float(b["reward"]))
        inter = client.export_interactions(b.get("style", "individual"), float(b.get("discount", 1.0)))
        store.pop(sid)
        reg.end_session(sid)
        return {"interactions": {k: serialize_value(v.to_tensor_dict()) for k, v in inter.items()}}

    app.state.registry, app.state.sessions, app.state.flags = reg, store, state
    return app


class GatewayInferenceEngine:
    """The trainer's handle on an inference service: the ``InferenceEngine`` calls that workflows and trainers
    make (``agenerate``, ``submit`` / ``wait`` / ``prepare_batch`` / ``rollout_batch`` through a local
    :class:`~areal_b200.infra.workflow_executor.WorkflowExecutor`, pause / continue, version) carried out over
    the gateway's routes, plus the session calls (``start_session`` / ``finish_session``) for multi-turn
    episodes that should stay on the engine holding their prefix. ``apost(url, body, headers) -> dict`` is the
    transport (default: aiohttp on the caller's loop).
    Reference: areal/experimental/inference_service/controller/controller.py (GatewayInferenceController)."""

    supports_images = False

    def __init__(self, config, gateway_url: str, token: str | None = None, apost=None):
        self.config, self.url, self.token = config, gateway_url.rstrip("/"), token
        self._apost = apost
        self._version = 0
        self._executor = None

    # ---------------------------------------------------------------- transport
    def _headers(self) -> dict[str, str]:
        return {"Authorization": f"Bearer {self.token}"} if self.token else {}

    async def _post(self, path: str, body: dict) -> dict:
        if self._apost is not None:
            return await self._apost(self.url + path, body, self._headers())
        from ..infra.utils.http import arequest_with_retry
        from ..infra.workflow_context import get_aiohttp_session

        session = await get_aiohttp_session()
        return await arequest_with_retry(session, "POST", self.url + path, json=body, headers=self._headers(),
                                         timeout=getattr(self.config, "request_timeout", 3600),
                                         max_retries=getattr(self.config, "request_retries", 3))

    def _post_sync(self, path: str, body: dict) -> dict:
        try:
            asyncio.get_running_loop()
        except RuntimeError:
            return asyncio.run(self._post_and_close(path, body))
        # called from a thread that runs a loop (a workflow): hop to a private loop in a helper thread
        box: dict[str, Any] = {}

        def run():
            try:
                box["v"] = asyncio.run(self._post_and_close(path, body))
            except BaseException as e:  # noqa: BLE001 - re-raised in the caller
                box["e"] = e

        t = threading.Thread(target=run, daemon=True)
        t.start()
        t.join()
        if "e" in box:
            raise box["e"]
        return box["v"]

    async def _post_and_close(self, path: str, body: dict) -> dict:
        try:
            return await self._post(path, body)
        finally:
            if self._apost is None:
                from ..infra.workflow_context import close_clients

                await close_clients()

    # ---------------------------------------------------------------- lifecycle
    def initialize(self, train_data_parallel_size: int | None = None, **_):
        from ..infra.workflow_executor import WorkflowExecutor

        self._executor = WorkflowExecutor(self.config, self).initialize(train_data_parallel_size)
        return self

    def destroy(self):
        if self._executor is not None:
            self._executor.destroy()
            self._executor = None

    # ---------------------------------------------------------------- generation
    async def agenerate(self, req, session_id: str | None = None):
        body = {"request": serialize_value(req)}
        sid = session_id or (getattr(req, "metadata", None) or {}).get("session_id")
        if sid:
            body["session_id"] = sid
        out = await self._post("/generate", body)
        return deserialize_value(out["response"])

    def generate(self, req, session_id: str | None = None):
        body = {"request": serialize_value(req)}
        if session_id:
            body["session_id"] = session_id
        return deserialize_value(self._post_sync("/generate", body)["response"])

    async def start_session(self, session_id: str | None = None) -> str:
        return (await self._post("/sessions/start", {"session_id": session_id} if session_id else {}))["session_id"]

    async def finish_session(self, session_id: str, reward: float | None = None) -> dict[str, Any]:
        """Ends the session; returns its trajectory (token ids, log-probs, loss mask, versions, reward)."""
        return (await self._post(f"/sessions/{session_id}/finish", {"reward": reward}))["trajectory"]

    # ---------------------------------------------------------------- control
    def pause_generation(self):
        self._post_sync("/pause", {})

    def continue_generation(self):
        self._post_sync("/continue", {})

    def set_version(self, version: int):
        self._version = int(version)
        self._post_sync("/set_version", {"version": int(version)})

    def get_version(self) -> int:
        return self._version

    # ---------------------------------------------------------------- workflow API
    def submit(self, data, workflow=None, workflow_kwargs=None, should_accept_fn=None, group_size=1, task_id=None,
               is_eval=False, **_) -> int:
        return self._executor.submit(data, workflow, workflow_kwargs, should_accept_fn, group_size, task_id=task_id,
                                     is_eval=is_eval)

    def wait(self, count: int, timeout: float | None = None, raise_timeout: bool = True):
        return self._executor.wait(count, timeout, raise_timeout)

    def wait_for_task(self, task_id: int, timeout: float | None = None, raise_timeout: bool = True):
        return self._executor.wait_for_task(task_id, timeout, raise_timeout)

    def rollout_batch(self, data, workflow=None, workflow_kwargs=None, should_accept_fn=None, group_size=1,
                      is_eval=False):
        return self._executor.rollout_batch(data, workflow, workflow_kwargs, should_accept_fn, group_size,
                                            is_eval=is_eval)

    def prepare_batch(self, dataloader, workflow=None, workflow_kwargs=None, should_accept_fn=None, group_size=1,
                      dynamic_bs=False):
        return self._executor.prepare_batch(dataloader, workflow, workflow_kwargs, should_accept_fn, group_size,
                                            dynamic_bs)

    def pause(self):
        self._executor.pause()

    def resume(self):
        self._executor.resume()

    def export_stats(self) -> dict[str, float]:
        return self._executor.export_stats() if self._executor is not None else {}
