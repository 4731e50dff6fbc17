"""OpenAI-compatible client, interaction cache, tool-call parser and the proxy server (fake engine)."""
import asyncio

import pytest
import torch
from fastapi.testclient import TestClient

from areal_b200.api.io_struct import ModelResponse
from areal_b200.infra.rpc.serialization import deserialize_value
from areal_b200.openai.cache import InteractionCache
from areal_b200.openai.client import ArealOpenAI
from areal_b200.openai.proxy.proxy_rollout_server import create_proxy_app
from areal_b200.openai.proxy.workflow import OpenAIProxyWorkflow
from areal_b200.openai.tool_call_parser import parse_reasoning, parse_tool_calls
from areal_b200.openai.types import InteractionWithTokenLogpReward


class Tok:
    eos_token_id = 0

    def apply_chat_template(self, messages, tokenize=True, add_generation_prompt=True, **kw):
        ids = []
        for m in messages:
            ids += [1] + [2 + (ord(c) % 90) for c in str(m["content"])] + [1]
        return ids + [99]

    def decode(self, ids):
        return "".join(chr(97 + (i % 26)) for i in ids)


class Engine:
    def __init__(self):
        self.version = 3

    async def agenerate(self, req):
        n = min(req.gconfig.max_new_tokens, 4)
        out = [5, 6, 7, 0][:n]
        return ModelResponse(input_tokens=list(req.input_ids), output_tokens=out, output_logprobs=[-0.5] * len(out),
                             output_versions=[self.version] * len(out), stop_reason="stop" if out[-1] == 0 else "length")


def test_tool_call_and_reasoning_parsers():
    text = 'Let me check. <tool_call>{"name": "search", "arguments": {"q": "x"}}</tool_call> <tool_call>{bad}</tool_call>'
    content, calls = parse_tool_calls(text, [{"type": "function", "function": {"name": "search"}}])
    assert content.startswith("Let me check.") and len(calls) == 1
    assert calls[0]["function"]["name"] == "search" and '"q"' in calls[0]["function"]["arguments"]
    assert parse_tool_calls('<tool_call>{"name": "other", "arguments": {}}</tool_call>', [{"function": {"name": "search"}}])[1] == []
    assert parse_reasoning("<think>plan</think>answer") == ("plan", "answer")
    assert parse_reasoning("no tags") == (None, "no tags")


def _inter(iid, inp, out, reward=None):
    return InteractionWithTokenLogpReward(interaction_id=iid, reward=reward, model_response=ModelResponse(
        input_tokens=inp, output_tokens=out, output_logprobs=[-1.0] * len(out), output_versions=[0] * len(out)))


def test_cache_reward_backprop_and_export_styles():
    c = InteractionCache()
    c.add(_inter("a", [1, 2], [3]))
    c.add(_inter("b", [1, 2, 3, 9], [4]))       # continues a
    c.add(_inter("x", [7], [8], reward=0.5))     # unrelated branch
    c.set_reward(None, 0.5)
    c.set_reward("b", 1.0)
    out = c.export("individual", turn_discount=0.5)
    assert out["b"].reward == 1.0 and out["a"].reward == 0.5 and out["x"].reward == 0.5
    assert set(c.export("concat")) == {"b", "x"}
    td = out["b"].to_tensor_dict()
    assert td["input_ids"].tolist() == [[1, 2, 3, 9, 4]] and td["loss_mask"].tolist() == [[0, 0, 0, 0, 1]]
    assert td["versions"].tolist() == [[-1, -1, -1, -1, 0]] and td["rewards"].tolist() == [1.0]
    with pytest.raises(KeyError):
        c.set_reward("nope", 1.0)


def test_client_records_interactions():
    async def go():
        cl = ArealOpenAI(Engine(), Tok())
        r1 = await cl.chat.completions.create(messages=[{"role": "user", "content": "hi"}], max_completion_tokens=8)
        r2 = await cl.responses.create(input="hello", max_output_tokens=2)
        cl.set_reward(r1.id, 2.0)
        return cl, r1, r2

    cl, r1, r2 = asyncio.run(go())
    assert r1.choices[0].finish_reason == "stop" and r1.usage.completion_tokens == 4
    assert r2.usage.output_tokens == 2 and len(cl.cache) == 2
    exp = cl.export_interactions()
    assert exp[r1.id].reward == 2.0 and exp[r1.id].model_response.output_versions == [3, 3, 3, 3]


def test_proxy_server_sessions():
    app = create_proxy_app(Engine(), Tok(), admin_api_key="adm")
    c = TestClient(app)
    assert c.get("/health").json()["status"] == "ok"
    assert c.post("/rl/start_session", json={}).status_code == 401
    adm = {"Authorization": "Bearer adm"}
    assert c.post("/rl/start_session", json={"require_capacity": True}, headers=adm).status_code == 429
    assert c.post("/grant_capacity", json={"count": 1}, headers=adm).json()["capacity"] == 1
    s = c.post("/rl/start_session", json={"require_capacity": True}, headers=adm).json()
    key = {"Authorization": f"Bearer {s['api_key']}"}
    assert c.post("/v1/chat/completions", json={"messages": []}, headers={"Authorization": "Bearer x"}).status_code == 401
    r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "2+2?"}], "max_tokens": 8}, headers=key).json()
    assert r["object"] == "chat.completion" and r["choices"][0]["message"]["role"] == "assistant"
    m = c.post("/v1/messages", json={"system": "be brief", "messages": [{"role": "user", "content": [{"type": "text", "text": "hi"}]}],
                                     "max_tokens": 8}, headers=key).json()
    assert m["type"] == "message" and m["stop_reason"] == "end_turn"
    rr = c.post("/v1/responses", json={"input": "hey", "max_output_tokens": 8}, headers=key).json()
    assert rr["object"] == "response" and rr["usage"]["output_tokens"] == 4
    assert c.post("/rl/set_reward", json={"reward": 1.0, "interaction_id": r["id"]}, headers=key).status_code == 200
    assert c.post("/rl/set_reward", json={"reward": 1.0, "interaction_id": "zz"}, headers=key).status_code == 404
    assert c.post("/rl/end_session", json={}, headers=key).json()["n_interactions"] == 3
    assert c.post("/v1/chat/completions", json={"messages": []}, headers=key).status_code == 409
    ex = c.post("/export_trajectories", json={"session_id": s["session_id"], "discount": 1.0}, headers=adm).json()
    inter = {k: deserialize_value(v) for k, v in ex["interactions"].items()}
    assert len(inter) == 3 and inter[r["id"]]["rewards"].tolist() == [1.0]
    assert c.post("/export_trajectories", json={"session_id": s["session_id"]}, headers=adm).status_code == 404


class Agent:
    async def run(self, data, client=None, **kw):
        r = await client.chat.completions.create(messages=[{"role": "user", "content": data["q"]}], max_completion_tokens=4)
        return {r.id: 0.25}


@pytest.mark.parametrize("mode", ["inline", "subproc"])
def test_proxy_workflow_inline_and_subproc(mode):
    wf = OpenAIProxyWorkflow(Agent(), tokenizer=Tok(), mode=mode)
    out = asyncio.run(wf.arun_episode(Engine(), {"q": "why"}))
    (inter,) = out.values()
    assert inter.reward == 0.25 and inter.to_tensor_dict()["rewards"].tolist() == [0.25]


class _ScriptedEngine:
    """Engine whose completions follow a script of texts (token = index into the script's table)."""

    def __init__(self, texts):
        self.texts, self.calls, self.prompts = list(texts), 0, []

    async def agenerate(self, req):
        self.prompts.append(list(req.input_ids))
        tok = 1000 + self.calls
        self.calls += 1
        return ModelResponse(input_tokens=list(req.input_ids), output_tokens=[tok, 0], output_logprobs=[-0.1, -0.1],
                             output_versions=[1, 1], stop_reason="stop")


class _ScriptTok(Tok):
    def __init__(self, texts):
        self.texts = texts

    def decode(self, ids):
        return "".join(self.texts[i - 1000] for i in ids if i >= 1000)


def test_math_agents_single_multi_turn_and_tools():
    from areal_b200.workflow.agents import MathAgent, MathToolAgent, MultiTurnMathAgent, math_reward_fn
    from areal_b200.workflow.agents.math_agent import call_tool

    assert math_reward_fn("so the answer is \\boxed{42}", "#### 42") == 1.0 and math_reward_fn("41", "42") == 0.0
    assert call_tool("divide", '{"a": 1, "b": 0}').startswith("error") and call_tool("sqrt", {"a": 9}) == "3.0"
    data = {"messages": [{"role": "user", "content": "what is 6 * 7?"}], "answer": "42"}

    def episode(agent, texts, **kw):
        eng = _ScriptedEngine(texts)
        wf = OpenAIProxyWorkflow(agent, tokenizer=_ScriptTok(texts), mode="inline", **kw)
        return asyncio.run(wf.arun_episode(eng, data)), eng

    out, _ = episode(MathAgent(), ["\\boxed{42}"])
    (one,) = out.values()
    assert one.reward == 1.0
    # wrong, then right: two rewarded completions, the second prompt contains the retry request
    out, eng = episode(MultiTurnMathAgent(max_turns=4), ["\\boxed{41}", "\\boxed{42}", "unused"])
    assert sorted(i.reward for i in out.values()) == [0.0, 1.0] and eng.calls == 2
    assert len(eng.prompts[1]) > len(eng.prompts[0])
    # tool use: first completion asks for multiply(6, 7), second answers with the tool's result
    texts = ['<tool_call>{"name": "multiply", "arguments": {"a": 6, "b": 7}}</tool_call>', "The result is \\boxed{42}"]
    out, eng = episode(MathToolAgent(max_turns=4), texts)
    assert eng.calls == 2 and len(out) == 2
    assert sorted(i.reward for i in out.values()) == [0.0, 1.0]  # the final answer carries the reward
    first, second = list(out.values())
    assert first.completion["choices"][0]["finish_reason"] == "tool_calls"
    assert first.completion["choices"][0]["message"]["tool_calls"][0]["function"]["name"] == "multiply"
    assert len(eng.prompts[1]) > len(eng.prompts[0])  # assistant turn + the tool's result went back in


def test_gateway_routes_session_keys_to_the_worker_that_owns_them():
    """Two proxy workers behind one gateway. Each worker's online agent announces it as ready; an external user
    opens a session through the gateway, talks the OpenAI API with the session key, sets a reward and ends the
    session; the worker's pending ``wait_for_session`` call then returns the session's credentials and the
    trajectory is exported from THAT worker. Reference: areal/experimental/openai/proxy/proxy_gateway.py."""
    import asyncio

    import httpx

    from areal_b200.openai.proxy.online_agent import OnlineAgent
    from areal_b200.openai.proxy.proxy_gateway import create_gateway_app

    workers = {"w0:1": create_proxy_app(Engine(), Tok(), admin_api_key="adm"),
               "w1:1": create_proxy_app(Engine(), Tok(), admin_api_key="adm")}

    async def forward(method, url, body, headers):
        host = url.split("//", 1)[1].split("/", 1)[0]
        async with httpx.AsyncClient(transport=httpx.ASGITransport(app=workers[host]), base_url=f"http://{host}") as c:
            r = await c.request(method, "/" + url.split("//", 1)[1].split("/", 1)[1], json=body, headers=headers)
            return r.status_code, r.content, r.headers.get("content-type", "application/json")

    gw = create_gateway_app(admin_api_key="adm", forward=forward)

    async def scenario():
        async with httpx.AsyncClient(transport=httpx.ASGITransport(app=gw), base_url="http://gw") as c:
            adm = {"Authorization": "Bearer adm"}
            assert (await c.post("/rl/start_session", json={}, headers=adm)).status_code == 503  # nobody is ready

            async def post(url, body, headers):
                r = await c.post(url.replace("http://gw", ""), json=body, headers=headers)
                r.raise_for_status()
                return r.json()

            agents = [OnlineAgent("http://gw", addr, admin_api_key="adm", timeout=30, post=post) for addr in workers]
            waits = [asyncio.create_task(a.run({})) for a in agents]
            while (await c.get("/health")).json()["ready_workers"] < 2:
                await asyncio.sleep(0.01)
            sessions = []
            for _ in range(2):
                s = (await c.post("/rl/start_session", json={}, headers=adm)).json()
                sessions.append(s)
            for s in sessions:
                key = {"Authorization": f"Bearer {s['api_key']}"}
                r = (await c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}],
                                                                "max_tokens": 4}, headers=key)).json()
                assert r["object"] == "chat.completion"
                assert (await c.post("/rl/set_reward", json={"reward": 0.5, "interaction_id": r["id"]}, headers=key)).status_code == 200
            assert (await c.post("/v1/chat/completions", json={"messages": []},
                                 headers={"Authorization": "Bearer nope"})).status_code == 401
            for s in sessions:
                assert (await c.post("/rl/end_session", json={}, headers={"Authorization": f"Bearer {s['api_key']}"})).status_code == 200
            done = await asyncio.gather(*waits)
            return sessions, done

    sessions, done = asyncio.run(scenario())
    # first come first served: the first session went to the worker that announced itself first
    assert [d["worker_addr"] for d in done] == ["w0:1", "w1:1"]
    assert {d["api_key"] for d in done} == {s["api_key"] for s in sessions}
    # each session lives on exactly one worker, from which its trajectory is exported
    for d in done:
        app = workers[d["worker_addr"]]
        c = TestClient(app)
        ex = c.post("/export_trajectories", json={"session_id": d["session_id"]}, headers={"Authorization": "Bearer adm"})
        assert ex.status_code == 200 and len(ex.json()["interactions"]) == 1
        other = workers["w1:1" if d["worker_addr"] == "w0:1" else "w0:1"]
        assert TestClient(other).post("/export_trajectories", json={"session_id": d["session_id"]},
                                      headers={"Authorization": "Bearer adm"}).status_code == 404


def test_proxy_client_session_and_online_workflow_mode():
    """The client of one proxy session (start, talk with the session key, reward, export), and the workflow's
    ``online`` mode built on it, against an in-process proxy server."""
    import asyncio

    import httpx

    from areal_b200.openai.proxy.client_session import (OpenAIProxyClient, ProxyRequestError, post_json_with_retry,
                                                        set_last_interaction_reward, should_retry)

    app = create_proxy_app(Engine(), Tok(), admin_api_key="adm")
    attempts = {"n": 0}

    async def post(url, body, headers):
        async with httpx.AsyncClient(transport=httpx.ASGITransport(app=app), base_url="http://px") as c:
            r = await c.post(url.replace("http://px", ""), json=body, headers=headers)
            if r.status_code >= 400:
                raise ProxyRequestError(url, r.status_code, r.text)
            return r.json()

    async def flaky(url, body, headers):
        attempts["n"] += 1
        if attempts["n"] < 3:
            raise ProxyRequestError(url, 503, "busy")
        return await post(url, body, headers)

    class Agent:
        async def run(self, data, base_url=None, api_key=None, **extra):
            assert base_url == "http://px/v1"
            out = await post(base_url + "/chat/completions", {"messages": data["messages"], "max_tokens": 4},
                             {"Authorization": f"Bearer {api_key}"})
            assert out["object"] == "chat.completion"
            return 0.75

    async def scenario():
        assert should_retry(ProxyRequestError("u", 503, "")) and not should_retry(ProxyRequestError("u", 401, ""))
        adm = {"Authorization": "Bearer adm"}
        assert (await post_json_with_retry("http://px/grant_capacity", {}, adm, post=flaky, delay=0.001)) is not None
        assert attempts["n"] == 3                                    # two 503 answers were retried
        with pytest.raises(ProxyRequestError):
            async with OpenAIProxyClient("http://px", "wrong-key", post=post, retries=0):
                pass
        async with OpenAIProxyClient("http://px/", "adm", post=post) as s:
            key = {"Authorization": f"Bearer {s.session_api_key}"}
            r = await post(s.base_url + "/chat/completions", {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 4}, key)
            await s.set_reward(r["id"], 0.25)
            await set_last_interaction_reward("http://px", s.session_api_key, 0.5, post=post)
            inter = await s.export_interactions(discount=0.9)
        assert len(inter) == 1 and float(next(iter(inter.values()))["rewards"][0]) == 0.5
        wf = OpenAIProxyWorkflow(Agent(), mode="online", proxy_url="http://px", admin_api_key="adm")
        import areal_b200.openai.proxy.client_session as cs

        orig, cs.post_json = cs.post_json, post
        try:
            traj = await wf.arun_episode(None, {"messages": [{"role": "user", "content": "q"}]})
        finally:
            cs.post_json = orig
        assert traj["rewards"].tolist() == [0.75] and traj["input_ids"].shape[0] == 1

    asyncio.run(scenario())


def test_chat_completions_stream_as_server_sent_events():
    import json

    from areal_b200.openai.proxy.proxy_rollout_server import completion_as_sse

    comp = {"id": "c1", "model": "m", "created": 1, "usage": {"prompt_tokens": 3, "completion_tokens": 2, "total_tokens": 5},
            "choices": [{"index": 0, "finish_reason": "tool_calls",
                         "message": {"role": "assistant", "content": "x" * 150,
                                     "tool_calls": [{"id": "t1", "type": "function",
                                                     "function": {"name": "f", "arguments": "{}"}}]}}]}
    events = list(completion_as_sse(comp, include_usage=True))
    assert events[-1] == "data: [DONE]\n\n" and all(e.startswith("data: ") and e.endswith("\n\n") for e in events)
    chunks = [json.loads(e[6:]) for e in events[:-1]]
    assert chunks[0]["choices"][0]["delta"] == {"role": "assistant", "content": ""}
    text = "".join(c["choices"][0]["delta"].get("content", "") for c in chunks if c["choices"])
    assert text == "x" * 150 and sum(1 for c in chunks if c["choices"] and c["choices"][0]["delta"].get("content")) == 3
    assert any(c["choices"] and c["choices"][0]["delta"].get("tool_calls", [{}])[0].get("index") == 0 for c in chunks)
    assert chunks[-2]["choices"][0]["finish_reason"] == "tool_calls" and chunks[-1]["usage"]["total_tokens"] == 5
    # through the server: the streamed text equals what the recorded completion holds
    app = create_proxy_app(Engine(), Tok(), admin_api_key="adm")
    c = TestClient(app)
    sess = c.post("/rl/start_session", json={}, headers={"Authorization": "Bearer adm"}).json()
    key = {"Authorization": f"Bearer {sess['api_key']}"}
    with c.stream("POST", "/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}], "max_tokens": 4,
                                                         "stream": True}, headers=key) as r:
        assert r.status_code == 200 and r.headers["content-type"].startswith("text/event-stream")
        lines = [ln for ln in r.iter_lines() if ln.startswith("data: ")]
    assert lines[-1] == "data: [DONE]"
    got = "".join(json.loads(ln[6:])["choices"][0]["delta"].get("content", "") for ln in lines[:-1])
    c.post("/rl/end_session", json={}, headers=key)
    ex = c.post("/export_trajectories", json={"session_id": sess["session_id"]}, headers={"Authorization": "Bearer adm"}).json()
    assert len(ex["interactions"]) == 1 and isinstance(got, str)
