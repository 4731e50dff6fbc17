"""Gateway / router / worker micro-services, wired together in-process: every outgoing POST of a
gateway is routed to the FastAPI app registered under the target address."""
import pytest
import torch
from fastapi.testclient import TestClient

from areal_b200.api.cli_args import GenerationHyperparameters
from areal_b200.api.io_struct import ModelRequest, ModelResponse
from areal_b200.infra.rpc.serialization import deserialize_value, serialize_value
from areal_b200.services import agent_service, data_service, inference_service, training_service, weight_update_service
from areal_b200.services.base import WorkerRegistry


class Net:
    """addr → TestClient; stands in for the network."""

    def __init__(self):
        self.apps = {}

    def add(self, addr, app):
        self.apps[addr] = TestClient(app)

    def post(self, url, body):
        addr, _, path = url[len("http://"):].partition("/")
        r = self.apps[addr].post("/" + path, json=body)
        if r.status_code >= 400:
            from areal_b200.infra.utils.http import HTTPRequestError

            raise HTTPRequestError(url, r.status_code, r.text)
        return r.json()


def test_registry_strategies_and_affinity():
    reg = WorkerRegistry("round_robin")
    for i in range(3):
        reg.register(f"w{i}", f"h{i}:1")
    assert [reg.pick().worker_id for _ in range(4)] == ["w0", "w1", "w2", "w0"]
    first = reg.pick("sess").worker_id
    assert all(reg.pick("sess").worker_id == first for _ in range(5))
    reg.mark_unhealthy(first)
    assert reg.pick("sess").worker_id != first
    ll = WorkerRegistry("least_loaded")
    a, b = ll.register("a", "x"), ll.register("b", "y")
    ll.acquire(a)
    assert ll.pick().worker_id == "b"
    with pytest.raises(ValueError):
        WorkerRegistry("random")


class SquaresDataset:
    def __init__(self, n=10):
        self.n = n

    def __len__(self):
        return self.n

    def __getitem__(self, i):
        return {"i": i, "sq": i * i}


def test_data_service_shards_fetches_and_prefetches():
    net = Net()
    for w in ("d0:1", "d1:1"):
        net.add(w, data_service.create_worker_app())
    gw = TestClient(data_service.create_gateway_app(token="s3cret", post=net.post))
    assert gw.post("/register", json={"worker_id": "d0", "addr": "d0:1"}).status_code == 401
    h = {"Authorization": "Bearer s3cret"}
    for i in range(2):
        assert gw.post("/register", json={"worker_id": f"d{i}", "addr": f"d{i}:1"}, headers=h).status_code == 200
    r = gw.post("/load", json={"name": "sq", "dataset": "tests.test_services.SquaresDataset",
                               "kwargs": serialize_value({"n": 10})}, headers=h)
    assert r.json()["len"] == 10
    ds = data_service.RDataset("gw", "sq", post=lambda path, body: gw.post(path, json=body, headers=h).json())
    assert len(ds) == 10 and ds[3] == {"i": 3, "sq": 9}
    assert [x["i"] for x in ds.fetch([7, 2, 5])] == [7, 2, 5]
    batches = [[0, 1], [2, 3], [4, 5], [6]]
    got = [[x["sq"] for x in b] for b in data_service.PrefetchingSampler(ds, batches, depth=2)]
    assert got == [[0, 1], [4, 9], [16, 25], [36]]


class EchoEngineApp:
    """Minimal stand-in for a worker RPC server hosting a rollout engine."""

    def __init__(self, name):
        from fastapi import FastAPI, Request

        self.name, self.calls, self.version = name, [], 0
        app = FastAPI()

        @app.post("/call")
        async def call(req: Request):
            b = await req.json()
            args = deserialize_value(b["args"])
            self.calls.append(b["method"])
            if b["method"] == "generate":
                mr = args[0]
                out = [t + 1 for t in mr.input_ids[-2:]]
                res = ModelResponse(input_tokens=list(mr.input_ids), output_tokens=out, output_logprobs=[-1.0] * len(out),
                                    output_versions=[self.version] * len(out), stop_reason="stop")
            elif b["method"] == "set_version":
                self.version = args[0]
                res = None
            else:
                res = None
            return {"result": serialize_value(res)}

        self.app = app


def test_inference_service_sessions_pause_and_versions():
    net = Net()
    engines = [EchoEngineApp("e0"), EchoEngineApp("e1")]
    for i, e in enumerate(engines):
        net.add(f"e{i}:1", e.app)
    gw = TestClient(inference_service.create_gateway_app(post=net.post))
    for i in range(2):
        gw.post("/register", json={"worker_id": f"e{i}", "addr": f"e{i}:1"})
    sid = gw.post("/sessions/start", json={}).json()["session_id"]
    req1 = ModelRequest(input_ids=[5, 6, 7], gconfig=GenerationHyperparameters(max_new_tokens=2))
    r1 = deserialize_value(gw.post("/generate", json={"session_id": sid, "request": serialize_value(req1)}).json()["response"])
    assert r1.output_tokens == [7, 8]
    gw.post("/set_version", json={"version": 4})
    req2 = ModelRequest(input_ids=[5, 6, 7, 7, 8, 9], gconfig=GenerationHyperparameters(max_new_tokens=2))
    gw.post("/generate", json={"session_id": sid, "request": serialize_value(req2)})
    # both turns of the session went to the same engine
    assert sorted(e.calls.count("generate") for e in engines) == [0, 2]
    traj = gw.post(f"/sessions/{sid}/finish", json={"reward": 1.0}).json()["trajectory"]
    assert traj["input_ids"] == [5, 6, 7, 7, 8, 9, 9, 10] and traj["loss_mask"] == [0, 0, 0, 1, 1, 0, 1, 1]
    assert traj["versions"] == [-1, -1, -1, 0, 0, -1, 4, 4] and traj["reward"] == 1.0
    assert gw.post("/pause", json={}).json()["paused"] and gw.get("/workers").json()["paused"]
    assert not gw.post("/continue", json={}).json()["paused"]
    assert all("pause_generation" in e.calls and "continue_generation" in e.calls for e in engines)


def test_training_service_splits_batches_and_merges():
    from tests.fake_engine import FakeTrainEngine
    from fastapi import FastAPI, Request

    net = Net()
    fakes = [FakeTrainEngine(), FakeTrainEngine()]

    def worker_app(eng):
        app = FastAPI()

        @app.post("/call")
        async def call(req: Request):
            b = await req.json()
            out = getattr(eng, b["method"])(*deserialize_value(b["args"]), **deserialize_value(b["kwargs"]))
            return {"result": serialize_value(out)}

        return app

    for i, f in enumerate(fakes):
        net.add(f"t{i}:1", worker_app(f))
    gw = TestClient(training_service.create_gateway_app(post=net.post))
    for i in range(2):
        gw.post("/register", json={"worker_id": f"t{i}", "addr": f"t{i}:1", "rank": i})
    B, L = 8, 6
    batch = {"input_ids": torch.arange(B * L).view(B, L), "attention_mask": torch.ones(B, L, dtype=torch.bool)}
    out = deserialize_value(gw.post("/call", json={"method": "forward_batch", "batch": serialize_value(batch),
                                                   "args": serialize_value([]), "kwargs": serialize_value({}),
                                                   "group_size": 2}).json()["result"])
    assert torch.equal(out, batch["input_ids"].float())  # rows came back in the original order
    gw.post("/call", json={"method": "set_version", "args": serialize_value([3]), "kwargs": serialize_value({})})
    assert all(f.version == 3 for f in fakes)


class CountingAgent:
    def __init__(self, bonus=0.0):
        self.bonus = bonus

    async def run(self, data, base_url=None, api_key=None):
        return {"reward": float(len(data["question"])) + self.bonus, "base_url": base_url}


def test_agent_service_runs_sessions_on_workers():
    net = Net()
    net.add("a0:1", agent_service.create_worker_app())
    gw = TestClient(agent_service.create_gateway_app(post=net.post))
    gw.post("/register", json={"worker_id": "a0", "addr": "a0:1"})
    sid = gw.post("/sessions/start", json={"base_url": "http://proxy/v1", "api_key": "k"}).json()["session_id"]
    r = gw.post(f"/sessions/{sid}/run", json={"agent": "tests.test_services.CountingAgent",
                                              "agent_kwargs": serialize_value({"bonus": 0.5}),
                                              "data": serialize_value({"question": "abcd"})})
    out = deserialize_value(r.json()["result"])
    assert out == {"reward": 4.5, "base_url": "http://proxy/v1"}
    assert gw.post(f"/sessions/{sid}/end", json={}).json()["runs"] == 1
    assert gw.post(f"/sessions/{sid}/run", json={"agent": "x.y"}).status_code == 404


def test_weight_update_service_round_and_metadata():
    net = Net()
    engines = [EchoEngineApp("e0"), EchoEngineApp("e1"), EchoEngineApp("e2")]
    for i, e in enumerate(engines):
        net.add(f"e{i}:1", e.app)
    gw = TestClient(weight_update_service.create_gateway_app(post=net.post))
    assert gw.post("/update_weights", json={}).status_code == 409
    for i in range(3):
        gw.post("/connect", json={"role": "inference", "rank": i, "addr": f"e{i}:1", "info": serialize_value({"ipc": i})})
    gw.post("/connect", json={"role": "train", "rank": 0, "addr": "e0:1"})
    gw.post("/connect", json={"role": "train", "rank": 1, "addr": "e1:1"})
    assert gw.get("/plan").json()["pairs"] == {"0": [0, 2], "1": [1]}
    gw.put("/weight_meta/exp/trial/v1", json={"path": "/ckpt/v1"})
    assert gw.get("/weight_meta/exp/trial/v1").json() == {"path": "/ckpt/v1"}
    assert gw.get("/weight_meta/none").status_code == 404
    r = gw.post("/update_weights", json={"mode": "disk", "meta": serialize_value({"path": "/ckpt/v1"})}).json()
    assert r["version"] == 1 and all(e.version == 1 for e in engines)
    for e in engines:
        i = e.calls.index
        assert i("pause_generation") < i("update_weights_from_disk") < i("set_version") < i("continue_generation")
    assert gw.get("/status").json()["version"] == 1
    assert weight_update_service.pair_ranks(2, 5) == {0: [0, 2, 4], 1: [1, 3]}


def test_gateway_inference_engine_runs_workflows_through_the_service():
    """The trainer-side engine object: a workflow's ``agenerate`` calls travel through the gateway to the engine
    workers; sessions keep their engine; pause / continue / version reach every worker."""
    import asyncio

    import httpx

    from areal_b200.api.cli_args import InferenceEngineConfig
    from areal_b200.api.workflow_api import RolloutWorkflow

    net = Net()
    engines = [EchoEngineApp("e0"), EchoEngineApp("e1")]
    for i, e in enumerate(engines):
        net.add(f"e{i}:1", e.app)
    app = inference_service.create_gateway_app(token="tok", post=net.post)

    async def apost(url, body, headers):
        async with httpx.AsyncClient(transport=httpx.ASGITransport(app=app), base_url="http://gw") as c:
            r = await c.post(url.replace("http://gw", ""), json=body, headers=headers)
            if r.status_code >= 400:
                raise RuntimeError(f"{r.status_code}: {r.text}")
            return r.json()

    asyncio.run(apost("http://gw/register", {"worker_id": "e0", "addr": "e0:1"}, {"Authorization": "Bearer tok"}))
    asyncio.run(apost("http://gw/register", {"worker_id": "e1", "addr": "e1:1"}, {"Authorization": "Bearer tok"}))
    cfg = InferenceEngineConfig(experiment_name="x", trial_name="y", max_concurrent_rollouts=8, consumer_batch_size=4,
                                max_head_offpolicyness=4)
    eng = inference_service.GatewayInferenceEngine(cfg, "http://gw", token="tok", apost=apost).initialize()
    try:
        bad = inference_service.GatewayInferenceEngine(cfg, "http://gw", token="wrong", apost=apost)
        with pytest.raises(RuntimeError, match="401"):
            bad.generate(ModelRequest(input_ids=[1], gconfig=GenerationHyperparameters(max_new_tokens=1)))

        class TwoTurns(RolloutWorkflow):
            async def arun_episode(self, engine, data):
                sid = await engine.start_session()
                g = GenerationHyperparameters(max_new_tokens=2)
                r1 = await engine.agenerate(ModelRequest(input_ids=data["ids"], gconfig=g), session_id=sid)
                ids2 = data["ids"] + r1.output_tokens + [99]
                await engine.agenerate(ModelRequest(input_ids=ids2, gconfig=g), session_id=sid)
                traj = await engine.finish_session(sid, reward=float(len(data["ids"])))
                n = len(traj["input_ids"])
                return dict(input_ids=torch.tensor(traj["input_ids"]).unsqueeze(0),
                            attention_mask=torch.ones(1, n, dtype=torch.bool),
                            loss_mask=torch.tensor(traj["loss_mask"]).unsqueeze(0),
                            logprobs=torch.tensor(traj["logprobs"]).unsqueeze(0),
                            versions=torch.tensor(traj["versions"]).unsqueeze(0),
                            rewards=torch.tensor([traj["reward"]]))

        batch = eng.rollout_batch([{"ids": [5, 6, 7]}, {"ids": [1, 2]}, {"ids": [3]}, {"ids": [4, 4, 4, 4]}],
                                  workflow=TwoTurns())
        assert batch["input_ids"].shape[0] == 4 and sorted(batch["rewards"].tolist()) == [1.0, 2.0, 3.0, 4.0]
        row = batch["rewards"].tolist().index(3.0)
        n = int(batch["attention_mask"][row].sum())
        assert batch["loss_mask"][row, :n].tolist() == [0, 0, 0, 1, 1, 0, 1, 1]
        # 8 generate calls, two per session, each session on one engine; round robin used both engines
        assert sum(e.calls.count("generate") for e in engines) == 8
        assert all(e.calls.count("generate") % 2 == 0 and e.calls.count("generate") > 0 for e in engines)
        eng.set_version(3)
        assert eng.get_version() == 3 and all(e.version == 3 for e in engines)
        eng.pause_generation()
        assert app.state.flags["paused"]
        eng.continue_generation()
        assert not app.state.flags["paused"]
        assert all("pause_generation" in e.calls and "continue_generation" in e.calls for e in engines)
    finally:
        eng.destroy()


def test_inference_gateway_speaks_the_chat_protocol_and_forwards_external_models():
    """Chat completions on the gateway: a session's turns stay on one engine and come back as training tensors;
    a request that names an external model goes to that provider untouched and is not recorded."""
    from tests.test_openai_proxy import Tok

    net = Net()
    engines = [EchoEngineApp("e0"), EchoEngineApp("e1")]
    for i, e in enumerate(engines):
        net.add(f"e{i}:1", e.app)
    sent = []

    def provider(url, body, headers):
        sent.append((url, body, headers))
        return {"id": "ext-1", "object": "chat.completion", "model": body["model"],
                "choices": [{"index": 0, "finish_reason": "stop", "message": {"role": "assistant", "content": "judge says yes"}}]}

    gw = TestClient(inference_service.create_gateway_app(
        post=net.post, tokenizer=Tok(), external_post=provider,
        external_models={"judge": {"url": "https://provider/v1/", "api_key": "sk-x", "model": "big-judge"}}))
    for i in range(2):
        gw.post("/register", json={"worker_id": f"e{i}", "addr": f"e{i}:1"})
    sid = gw.post("/sessions/start", json={}).json()["session_id"]
    msgs = [{"role": "user", "content": "hi"}]
    c1 = gw.post("/v1/chat/completions", json={"messages": msgs, "session_id": sid, "max_tokens": 4}).json()
    assert c1["object"] == "chat.completion" and c1["choices"][0]["message"]["role"] == "assistant"
    msgs += [c1["choices"][0]["message"], {"role": "user", "content": "more"}]
    c2 = gw.post("/v1/chat/completions", json={"messages": msgs, "max_tokens": 4}, headers={"X-Session-Id": sid}).json()
    assert sorted(e.calls.count("generate") for e in engines) == [0, 2]            # one engine served both turns
    ext = gw.post("/v1/chat/completions", json={"messages": msgs, "model": "judge", "session_id": sid, "temperature": 0}).json()
    assert ext["choices"][0]["message"]["content"] == "judge says yes"
    url, body, headers = sent[0]
    assert url == "https://provider/v1/chat/completions" and body["model"] == "big-judge" and "session_id" not in body
    assert headers == {"Authorization": "Bearer sk-x"} and sum(e.calls.count("generate") for e in engines) == 2
    out = gw.post(f"/sessions/{sid}/export_chat", json={"reward": 1.0, "rewards": {c1["id"]: 0.25}, "discount": 1.0}).json()
    inter = {k: deserialize_value(v) for k, v in out["interactions"].items()}
    assert set(inter) == {c1["id"], c2["id"]}
    assert float(inter[c2["id"]]["rewards"][0]) == 1.0 and float(inter[c1["id"]]["rewards"][0]) == 0.25
    assert int(inter[c1["id"]]["loss_mask"].sum()) == 2                            # the echo engine produced two tokens
    assert gw.post(f"/sessions/{sid}/export_chat", json={}).status_code == 404
    assert gw.post("/v1/chat/completions", json={"messages": msgs, "session_id": "nope"}).status_code == 404
    plain = TestClient(inference_service.create_gateway_app(post=net.post))
    assert plain.post("/v1/chat/completions", json={"messages": msgs}).status_code == 501


def sft_token_weight(mb):
    return float(mb["loss_mask"].sum())


def sft_mean_loss(logprobs, entropy, mb):
    # position t holds log p(x[t+1] | x[<=t]): the mask of the NEXT token applies (a sequence's first token is
    # never a target, so rolling the packed mask also clears every sequence's last position)
    m = torch.roll(mb["loss_mask"], -1).float()
    return -(logprobs * m).sum() / m.sum().clamp(min=1)


def test_gateway_train_engine_drives_real_engines_through_the_service(tmp_path):
    """The trainer-side handle of a training service over two real (CPU) train engines: a step through the
    gateway equals the step of one engine on the whole batch, loss functions travel by import path, and an
    evaluation batch that does not divide over the workers is padded and trimmed."""
    from fastapi import FastAPI, Request

    from areal_b200.api.cli_args import OptimizerConfig, TrainEngineConfig
    from areal_b200.engine.train_engine import B200TrainEngine

    def make_engine():
        e = B200TrainEngine(TrainEngineConfig(experiment_name="e", trial_name="t", path="", init_from_scratch=True,
                                              dtype="float32", model_preset="tiny-qwen2",
                                              optimizer=OptimizerConfig(lr=1e-3, warmup_steps_proportion=0.0)))
        e.create_process_group()
        e.initialize(seed=5)
        return e

    def worker_app(eng):
        app = FastAPI()

        @app.post("/call")
        async def call(req: Request):
            b = await req.json()
            out = getattr(eng, b["method"])(*deserialize_value(b["args"]), **deserialize_value(b["kwargs"]))
            return {"result": serialize_value(out if not isinstance(out, B200TrainEngine) else None)}

        return app

    net = Net()
    engines = [make_engine(), make_engine()]
    for i, e in enumerate(engines):
        net.add(f"t{i}:1", worker_app(e))
    gw_app = training_service.create_gateway_app(token="tok", post=net.post)
    gw = TestClient(gw_app)
    hdr = {"Authorization": "Bearer tok"}
    for i in range(2):
        gw.post("/register", json={"worker_id": f"t{i}", "addr": f"t{i}:1", "rank": i}, headers=hdr)
    client = training_service.GatewayTrainEngine(
        "http://gw", token="tok", post=lambda url, body, headers: gw.post(url.replace("http://gw", ""), json=body, headers=headers).json())
    assert client.n_workers() == 2
    g = torch.Generator().manual_seed(0)
    B, L = 5, 12
    batch = {"input_ids": torch.randint(0, 1000, (B, L), generator=g), "attention_mask": torch.ones(B, L, dtype=torch.bool),
             "loss_mask": torch.ones(B, L, dtype=torch.int32)}
    batch["loss_mask"][:, 0] = 0
    lp = client.forward_batch(batch)                                  # 5 samples over 2 workers: padded to 6, trimmed
    ref = make_engine()
    assert lp.shape == (B, L) and torch.allclose(lp, ref.forward_batch(batch), atol=1e-5)
    # these two workers are separate processes without a common process group, so each scores its own share (in a
    # deployment they are data-parallel ranks and all-reduce); the gateway reports the first rank's figure
    from areal_b200.infra.controller.train_controller import dispatch_batch, pad_batch_for_dispatch

    share0 = dispatch_batch(pad_batch_for_dispatch(batch, 2)[0], 2)[0][0]
    ev = client.eval_batch(batch, sft_mean_loss, sft_token_weight)
    assert abs(float(ev) - float(ref.eval_batch(share0, sft_mean_loss, sft_token_weight))) < 1e-4
    with pytest.raises(ValueError, match="importable"):
        client.train_batch(batch, lambda *a: 0.0, sft_token_weight)
    client.set_version(4)
    assert client.get_version() == 4 and all(e.get_version() == 4 for e in engines)
    for e in engines + [ref]:
        e.destroy()


def test_agent_service_speaks_the_responses_protocol_and_keeps_the_conversation():
    """``/v1/responses``: ``user`` names the conversation, the gateway keeps its history and hands it to the agent on
    the session's worker; the example agent calls its chat endpoint, runs the calculator the model asks for, and its
    answer comes back as a ``response`` object."""
    import os
    import sys

    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from examples.agent_service import agent as agent_mod

    seen = []

    def fake_chat(url, body):
        seen.append((url, [dict(m) for m in body["messages"]]))
        last = body["messages"][-1]["content"]
        if last.startswith("<result>"):
            text = f"The answer is {last[8:-9]}."
        elif "17 * 23" in last:
            text = "Let me compute. <calc>17 * 23</calc> (waiting)"
        else:
            text = f"You have sent {sum(m['role'] == 'user' for m in body['messages'])} messages."
        return {"choices": [{"message": {"role": "assistant", "content": text}}]}

    orig = agent_mod.ChatAgent.__init__
    agent_mod.ChatAgent.__init__ = lambda self, **kw: orig(self, post=fake_chat, **kw)
    try:
        net = Net()
        net.add("a0:1", agent_service.create_worker_app())
        net.add("a1:1", agent_service.create_worker_app())
        gw = TestClient(agent_service.create_gateway_app(post=net.post, agent="examples.agent_service.agent.ChatAgent",
                                                         agent_kwargs={"model": "m"}, base_url="http://llm/v1"))
        for i in range(2):
            gw.post("/register", json={"worker_id": f"a{i}", "addr": f"a{i}:1"})
        r = gw.post("/v1/responses", json={"input": [{"type": "message", "content": "What is 17 * 23?"}],
                                           "user": "alice", "model": "m"}).json()
        assert r["object"] == "response" and r["output_text"] == "The answer is 391."
        assert r["output"][0]["content"][0] == {"type": "output_text", "text": "The answer is 391.", "annotations": []}
        assert r["metadata"]["tool_calls"] == 1 and seen[0][0] == "http://llm/v1/chat/completions"
        # the second turn of the same user sees the first; another user starts empty
        r2 = gw.post("/v1/responses", json={"input": "and how many messages so far?", "user": "alice"}).json()
        assert r2["output_text"] == "You have sent 2 messages."
        r3 = gw.post("/v1/responses", json={"input": [{"type": "message", "role": "user",
                                                       "content": [{"type": "input_text", "text": "hello"}]}],
                                            "user": "bob"}).json()
        assert r3["output_text"] == "You have sent 1 messages."
        assert len(gw.app.state.conversations["alice"]) == 4
        assert gw.post("/v1/conversations/alice/reset", json={}).json()["dropped_messages"] == 4
        assert gw.post("/v1/responses", json={"input": [], "user": "bob"}).status_code == 400
    finally:
        agent_mod.ChatAgent.__init__ = orig
    bare = TestClient(agent_service.create_gateway_app(post=net.post))
    assert bare.post("/v1/responses", json={"input": "hi"}).status_code == 501
    assert agent_mod.calculate("2 ** 10 - 24") == "1000" and agent_mod.calculate("__import__('os')").startswith("error")
