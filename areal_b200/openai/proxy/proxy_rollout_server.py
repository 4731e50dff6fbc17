"""OpenAI / Anthropic compatible HTTP proxy in front of a rollout engine, with RL sessions.

Admin endpoints (``Authorization: Bearer <admin key>``): ``POST /grant_capacity``,
``POST /rl/start_session`` → ``{session_id, api_key}``, ``POST /export_trajectories``.
Session endpoints (``Authorization: Bearer <session api key>``):
``POST /v1/chat/completions``, ``POST /v1/responses``, ``POST /v1/messages``,
``POST /rl/set_reward``, ``POST /rl/end_session``. ``GET /health`` is open.

Every completion made with a session key is recorded (token ids, logprobs, policy
versions) in that session's :class:`InteractionCache`; ``export_trajectories``
applies the turn discount and returns the session's training samples
(role of areal/experimental/openai/proxy/proxy_rollout_server.py).
"""

from __future__ import annotations

import asyncio
import secrets
import time
import uuid

from fastapi import FastAPI, HTTPException, Request

from ...api.cli_args import GenerationHyperparameters
from ...infra.rpc.serialization import serialize_value
from ..client import ArealOpenAI


class Session:
    def __init__(self, session_id: str, api_key: str, client: ArealOpenAI, task_id: str | None):
        self.session_id, self.api_key, self.client, self.task_id = session_id, api_key, client, task_id
        self.started = time.time()
        self.ended: float | None = None
        self.finished = asyncio.Event()


def completion_as_sse(comp: dict, include_usage: bool = False, piece_chars: int = 64):
    """A finished chat completion as the event stream of ``stream: true``: a role chunk, the text in pieces, the
    tool calls, a chunk with the finish reason (then one with the usage when asked for) and ``[DONE]``. The
    rollout engine delivers whole responses (the training record needs every token's log-prob and version), so
    streaming clients get the same content re-cut into chunks rather than tokens as they are sampled."""
    import json as _json

    choice = comp["choices"][0]
    msg = choice["message"]
    base = {"id": comp["id"], "object": "chat.completion.chunk", "created": comp.get("created", int(time.time())),
            "model": comp.get("model", "default")}

    def event(delta: dict, finish=None, **extra) -> str:
        body = dict(base, choices=[{"index": 0, "delta": delta, "finish_reason": finish}], **extra)
        return "data: " + _json.dumps(body) + "\n\n"

    yield event({"role": "assistant", "content": ""})
    text = msg.get("content") or ""
    for i in range(0, len(text), piece_chars):
        yield event({"content": text[i:i + piece_chars]})
    if msg.get("reasoning_content"):
        yield event({"reasoning_content": msg["reasoning_content"]})
    for i, call in enumerate(msg.get("tool_calls") or []):
        yield event({"tool_calls": [dict(call, index=i)]})
    yield event({}, finish=choice.get("finish_reason", "stop"))
    if include_usage and comp.get("usage"):
        yield "data: " + _json.dumps(dict(base, choices=[], usage=comp["usage"])) + "\n\n"
    yield "data: [DONE]\n\n"


def create_proxy_app(engine, tokenizer, admin_api_key: str = "areal-admin-key",
                     gconfig: GenerationHyperparameters | None = None, tool_call_parser: str = "qwen",
                     reasoning_parser: str | None = None, session_timeout_seconds: int = 3600,
                     engine_max_tokens: int | None = None, processor=None) -> FastAPI:
    """``processor``: the HF processor of a vision-language model; with it ``image_url`` message parts are
    expanded on this side (see ``ArealOpenAI``)."""
    app = FastAPI()
    sessions: dict[str, Session] = {}
    by_key: dict[str, Session] = {}
    state = {"capacity": 0}

    def bearer(req: Request) -> str:
        auth = req.headers.get("authorization") or req.headers.get("x-api-key") or ""
        return auth[7:] if auth.lower().startswith("bearer ") else auth

    def require_admin(req: Request):
        if bearer(req) != admin_api_key:
            raise HTTPException(status_code=401, detail="admin key required")

    def session_of(req: Request) -> Session:
        s = by_key.get(bearer(req))
        if s is None:
            raise HTTPException(status_code=401, detail="unknown session key")
        if s.ended is not None:
            raise HTTPException(status_code=409, detail="session has ended")
        if time.time() - s.started > session_timeout_seconds:
            raise HTTPException(status_code=408, detail="session expired")
        return s

    @app.get("/health")
    def health():
        return {"status": "ok", "sessions": len(sessions), "capacity": state["capacity"]}

    @app.post("/grant_capacity")
    async def grant_capacity(req: Request):
        require_admin(req)
        body = await req.json() if await req.body() else {}
        state["capacity"] += int(body.get("count", 1))
        return {"capacity": state["capacity"]}

    @app.post("/rl/start_session")
    async def start_session(req: Request):
        require_admin(req)
        body = await req.json() if await req.body() else {}
        if body.get("require_capacity", False):
            if state["capacity"] <= 0:
                raise HTTPException(status_code=429, detail="no capacity granted")
            state["capacity"] -= 1
        sid = uuid.uuid4().hex
        key = "sk-sess-" + secrets.token_hex(16)
        client = ArealOpenAI(engine, tokenizer, gconfig, tool_call_parser, reasoning_parser,
                             engine_max_tokens=engine_max_tokens, processor=processor)
        s = Session(sid, key, client, body.get("task_id"))
        sessions[sid] = s
        by_key[key] = s
        return {"session_id": sid, "api_key": key}

    @app.post("/v1/chat/completions")
    async def chat_completions(req: Request):
        s = session_of(req)
        b = await req.json()
        comp = await s.client._complete(b["messages"], model=b.get("model", "default"), tools=b.get("tools"),
                                        max_new=b.get("max_completion_tokens") or b.get("max_tokens"),
                                        temperature=b.get("temperature"), top_p=b.get("top_p"), stop=b.get("stop"),
                                        as_dict=True)
        if not b.get("stream"):
            return comp
        from fastapi.responses import StreamingResponse

        include_usage = bool((b.get("stream_options") or {}).get("include_usage"))
        return StreamingResponse(completion_as_sse(comp, include_usage), media_type="text/event-stream")

    @app.post("/v1/responses")
    async def responses(req: Request):
        s = session_of(req)
        b = await req.json()
        inp = b.get("input")
        messages = [{"role": "user", "content": inp}] if isinstance(inp, str) else list(inp or [])
        if b.get("instructions"):
            messages = [{"role": "system", "content": b["instructions"]}] + messages
        comp = await s.client._complete(messages, model=b.get("model", "default"), tools=b.get("tools"),
                                        max_new=b.get("max_output_tokens"), temperature=b.get("temperature"),
                                        top_p=b.get("top_p"), stop=None, as_dict=True)
        text = comp["choices"][0]["message"]["content"]
        return {"id": comp["id"], "object": "response", "model": comp["model"], "status": "completed",
                "output_text": text,
                "output": [{"type": "message", "role": "assistant", "content": [{"type": "output_text", "text": text}]}],
                "usage": {"input_tokens": comp["usage"]["prompt_tokens"],
                          "output_tokens": comp["usage"]["completion_tokens"]}}

    @app.post("/v1/messages")
    async def anthropic_messages(req: Request):
        s = session_of(req)
        b = await req.json()
        messages = []
        if b.get("system"):
            sys_txt = b["system"] if isinstance(b["system"], str) else "".join(p.get("text", "") for p in b["system"])
            messages.append({"role": "system", "content": sys_txt})
        for m in b.get("messages", []):
            c = m["content"]
            if isinstance(c, list):
                c = "".join(p.get("text", "") for p in c if p.get("type") == "text")
            messages.append({"role": m["role"], "content": c})
        comp = await s.client._complete(messages, model=b.get("model", "default"), tools=None,
                                        max_new=b.get("max_tokens"), temperature=b.get("temperature"),
                                        top_p=b.get("top_p"), stop=b.get("stop_sequences"), as_dict=True)
        finish = comp["choices"][0]["finish_reason"]
        return {"id": comp["id"], "type": "message", "role": "assistant", "model": comp["model"],
                "content": [{"type": "text", "text": comp["choices"][0]["message"]["content"]}],
                "stop_reason": "end_turn" if finish == "stop" else "max_tokens",
                "usage": {"input_tokens": comp["usage"]["prompt_tokens"],
                          "output_tokens": comp["usage"]["completion_tokens"]}}

    @app.post("/rl/set_reward")
    async def set_reward(req: Request):
        s = session_of(req)
        b = await req.json()
        try:
            s.client.set_reward(b.get("interaction_id"), float(b["reward"]))
        except KeyError as e:
            raise HTTPException(status_code=404, detail=str(e))
        return {"status": "ok"}

    @app.post("/rl/end_session")
    async def end_session(req: Request):
        s = session_of(req)
        s.ended = time.time()
        s.finished.set()
        return {"status": "ok", "n_interactions": len(s.client.cache)}

    @app.post("/export_trajectories")
    async def export_trajectories(req: Request):
        require_admin(req)
        b = await req.json()
        s = sessions.get(b["session_id"])
        if s is None:
            raise HTTPException(status_code=404, detail="unknown session")
        if b.get("wait", False) and s.ended is None:
            try:
                await asyncio.wait_for(s.finished.wait(), timeout=float(b.get("timeout", 600)))
            except asyncio.TimeoutError:
                raise HTTPException(status_code=408, detail="session did not end in time")
        inter = s.client.export_interactions(b.get("style", "individual"), float(b.get("discount", 1.0)))
        out = {k: serialize_value(v.to_tensor_dict()) for k, v in inter.items()}
        if b.get("remove", True):
            sessions.pop(s.session_id, None)
            by_key.pop(s.api_key, None)
        return {"session_id": s.session_id, "interactions": out}

    app.state.sessions = sessions
    return app
