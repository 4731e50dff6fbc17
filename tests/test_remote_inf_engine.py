"""RemoteInfEngine against real localhost servers of the native engine (CPU model): discovery,
routing with request affinity, interruptible generation across a pause, control fan-out, disk weight
update, and the wire format of the other backends."""
import asyncio
import socket
import threading
import time

import pytest
import torch
import uvicorn

from areal_b200.api.cli_args import GenerationHyperparameters, InferenceEngineConfig, NativeRolloutConfig
from areal_b200.api.io_struct import ModelRequest, WeightUpdateMeta
from areal_b200.engine.native_server import create_app
from areal_b200.engine.rollout_engine import NativeRolloutEngine
from areal_b200.infra.remote_inf_engine import NativeBackend, RemoteInfEngine, SGLangBackend, VLLMBackend


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


class _Server:
    def __init__(self, seed=0):
        cfg = InferenceEngineConfig(experiment_name="e", trial_name="t", backend="native:d1", max_concurrent_rollouts=16,
                                    consumer_batch_size=4,
                                    native=NativeRolloutConfig(model_preset="tiny-qwen2", context_length=256, max_num_seqs=8,
                                                               max_num_batched_tokens=512, num_kv_blocks=64, seed=seed,
                                                               cuda_graph=False))
        self.engine = NativeRolloutEngine(cfg).initialize(device="cpu")
        self.port = _free_port()
        self.server = uvicorn.Server(uvicorn.Config(create_app(self.engine), host="127.0.0.1", port=self.port,
                                                    log_level="error"))
        self.thread = threading.Thread(target=self.server.run, daemon=True)
        self.thread.start()
        self.addr = f"127.0.0.1:{self.port}"

    def stop(self):
        self.server.should_exit = True
        self.thread.join(timeout=10)
        self.engine.destroy()


@pytest.fixture()
def servers():
    ss = [_Server(0), _Server(0)]
    yield ss
    for s in ss:
        s.stop()


def _client(addrs, **kw):
    cfg = InferenceEngineConfig(experiment_name="e", trial_name="t", backend="native:d2", max_concurrent_rollouts=16,
                                consumer_batch_size=4, setup_timeout=30.0, request_timeout=60.0, **kw)
    return RemoteInfEngine(cfg).initialize(addr=addrs)


def test_generation_routing_and_control(servers, tmp_path):
    cli = _client([s.addr for s in servers])
    try:
        prompt = torch.randint(0, 1000, (20,), generator=torch.Generator().manual_seed(1)).tolist()
        gc = GenerationHyperparameters(max_new_tokens=12, greedy=True, ignore_eos=True)
        # greedy output over HTTP == greedy output of the engine itself
        r = cli.generate(ModelRequest(rid="a", input_ids=prompt, gconfig=gc))
        direct = servers[0].engine.generate(ModelRequest(rid="x", input_ids=prompt, gconfig=gc))
        assert r.output_tokens == direct.output_tokens and len(r.output_logprobs) == 12
        assert r.stop_reason == "length" and r.output_versions == [0] * 12
        # request-id affinity and round-robin
        assert cli.choose_server("a") == cli.choose_server("a")
        assert {cli.choose_server(f"r{i}") for i in range(4)} == {s.addr for s in servers}
        # version fan-out reaches every server and tags later tokens
        cli.set_version(5)
        assert all(s.engine.get_version() == 5 for s in servers)
        r2 = cli.generate(ModelRequest(rid="b", input_ids=prompt, gconfig=gc))
        assert r2.output_versions == [5] * 12
        # pause / continue fan-out
        cli.pause_generation()
        assert all(s.engine._paused.is_set() for s in servers)
        cli.continue_generation()
        assert not any(s.engine._paused.is_set() for s in servers)
        # weights from a checkpoint directory: both servers load it and answer with the new model
        from areal_b200.models.qwen import build_model
        from areal_b200.utils.hf_io import save_hf_checkpoint

        other = build_model(servers[0].engine.model_config, dtype=torch.float32, seed=123)
        save_hf_checkpoint(other, servers[0].engine.model_config, str(tmp_path / "ckpt"))
        cli.update_weights_from_disk(WeightUpdateMeta(type="disk", path=str(tmp_path / "ckpt"), version=6)).result(60)
        assert cli.get_version() == 6 and all(s.engine.get_version() == 6 for s in servers)
        r3 = cli.generate(ModelRequest(rid="c", input_ids=prompt, gconfig=gc))
        assert r3.output_tokens != r.output_tokens and r3.output_versions == [6] * 12
        with pytest.raises(NotImplementedError):
            cli.update_weights_from_distributed(WeightUpdateMeta(type="xccl"), [])
    finally:
        cli.destroy()


def test_generation_survives_a_pause(servers):
    """A weight update in the middle of a long generation: the server aborts the request, the client
    re-issues prompt + partial output, and the tokens carry the version that produced them."""
    cli = _client([servers[0].addr])
    try:
        prompt = list(range(10, 40))
        gc = GenerationHyperparameters(max_new_tokens=150, greedy=True, ignore_eos=True)

        async def go():
            task = asyncio.ensure_future(cli.agenerate(ModelRequest(rid="long", input_ids=prompt, gconfig=gc)))
            loop = asyncio.get_running_loop()
            await asyncio.sleep(0.3)
            await loop.run_in_executor(None, cli.pause_generation)
            await loop.run_in_executor(None, lambda: cli.set_version(1))
            await asyncio.sleep(0.1)
            await loop.run_in_executor(None, cli.continue_generation)
            try:
                return await task
            finally:
                from areal_b200.infra.workflow_context import close_clients

                await close_clients()

        r = asyncio.run(go())
        assert len(r.output_tokens) == 150 and r.stop_reason == "length"
        assert set(r.output_versions) <= {0, 1} and r.output_versions == sorted(r.output_versions)
        # same weights before and after: the interrupted run equals an uninterrupted one
        ref = servers[1].engine.generate(ModelRequest(rid="ref", input_ids=prompt, gconfig=gc))
        assert r.output_tokens == ref.output_tokens
    finally:
        cli.destroy()


def test_workflow_api_over_http(servers):
    from areal_b200.workflow.rlvr import RLVRWorkflow

    cli = _client([s.addr for s in servers])
    try:
        gc = GenerationHyperparameters(max_new_tokens=6, greedy=False, temperature=1.0, ignore_eos=True)
        wf = RLVRWorkflow(reward_fn=lambda *a, **k: 1.0, gconfig=gc, reward_in_process=True)
        data = [{"input_ids": [3, 4, 5, 6 + i]} for i in range(4)]
        batch = cli.rollout_batch(data, workflow=wf, group_size=2)
        assert batch["input_ids"].shape[0] == 8 and float(batch["rewards"].sum()) == 8.0
    finally:
        cli.destroy()


def test_discovery_through_name_resolve_and_env(servers, monkeypatch):
    from areal_b200.utils import name_resolve, names

    name_resolve.reset()
    for i, s in enumerate(servers):
        name_resolve.add(names.gen_server("e", "t", i), s.addr, replace=True)
    cfg = InferenceEngineConfig(experiment_name="e", trial_name="t", backend="native:d2", consumer_batch_size=2,
                                setup_timeout=10.0)
    cli = RemoteInfEngine(cfg).initialize()
    assert sorted(cli.addresses) == sorted(s.addr for s in servers)
    cli.destroy()
    monkeypatch.setenv("AREAL_LLM_SERVER_ADDRS", servers[1].addr)
    cli = RemoteInfEngine(cfg).initialize()
    assert cli.addresses == [servers[1].addr]
    cli.destroy()
    name_resolve.reset()
    monkeypatch.delenv("AREAL_LLM_SERVER_ADDRS")
    cfg2 = InferenceEngineConfig(experiment_name="none", trial_name="t", backend="native:d1", setup_timeout=0.5)
    with pytest.raises(TimeoutError):
        RemoteInfEngine(cfg2).initialize()


def test_backend_wire_formats():
    gc = GenerationHyperparameters(max_new_tokens=64, temperature=0.7, top_p=0.9, top_k=20, stop_token_ids=[2], min_new_tokens=3)
    req = ModelRequest(rid="r", input_ids=[1, 2, 3], gconfig=gc)
    sg = SGLangBackend().build_generation_request(req, [1, 2, 3, 9], 60)
    assert sg.endpoint == "/generate" and sg.payload["input_ids"] == [1, 2, 3, 9] and sg.payload["return_logprob"]
    sp = sg.payload["sampling_params"]
    assert sp["max_new_tokens"] == 60 and sp["temperature"] == 0.7 and sp["stop_token_ids"] == [2] and sp["min_new_tokens"] == 3
    res, ver = SGLangBackend().parse_generation_response(
        {"meta_info": {"finish_reason": {"type": "abort"}, "output_token_logprobs": [[-0.5, 11, None], [-1.5, 12, None]]}})
    assert res.output_tokens == [11, 12] and res.output_logprobs == [-0.5, -1.5] and res.stop_reason == "abort" and ver is None
    greedy = ModelRequest(rid="g", input_ids=[1], gconfig=GenerationHyperparameters(greedy=True, max_new_tokens=4))
    assert SGLangBackend().build_generation_request(greedy, [1], 4).payload["sampling_params"]["temperature"] == 0.0
    vl = VLLMBackend().build_generation_request(req, [1, 2, 3], 64)
    assert vl.endpoint == "/v1/completions" and vl.payload["prompt"] == [1, 2, 3] and vl.payload["return_tokens_as_token_ids"]
    res, _ = VLLMBackend().parse_generation_response(
        {"choices": [{"finish_reason": "length", "logprobs": {"tokens": ["token_id:7", "token_id:8"], "token_logprobs": [-0.1, -0.2]}}]})
    assert res.output_tokens == [7, 8] and res.stop_reason == "length"
    assert VLLMBackend().pause().endpoint == "/areal_pause_generation"
    assert NativeBackend().set_version(3).payload == {"version": 3} and SGLangBackend().set_version(3) is None


def test_launch_server_subprocess():
    """`launch_server` starts `python -m areal_b200.engine.native_server` and the client talks to it."""
    cfg = InferenceEngineConfig(experiment_name="e", trial_name="t", backend="native:d1", consumer_batch_size=1,
                                setup_timeout=120.0, request_timeout=60.0)
    cli = RemoteInfEngine(cfg)
    try:
        info = cli.launch_server(dict(model_preset="tiny-qwen2", device="cpu", disable_cuda_graph=True, num_kv_blocks=32,
                                      context_length=128, max_num_seqs=4, max_num_batched_tokens=256))
        assert info.process.poll() is None and cli.addresses == [f"{info.host}:{info.port}"]
        cli.initialize(addr=cli.addresses)
        r = cli.generate(ModelRequest(rid="s", input_ids=[5, 6, 7, 8],
                                      gconfig=GenerationHyperparameters(max_new_tokens=4, greedy=True, ignore_eos=True)))
        assert len(r.output_tokens) == 4
    finally:
        cli.destroy()
    assert info.process.poll() is not None  # torn down with the client


def test_trainer_with_external_http_server(tmp_path, monkeypatch):
    """PPOTrainer against a rollout server reached over HTTP: generation through RemoteInfEngine, weights
    through a checkpoint directory, versions bumped on the server after every step."""
    from areal_b200.api.cli_args import (GRPOConfig, MicroBatchSpec, NormConfig, OptimizerConfig, PPOActorConfig,
                                         _propagate_names)
    from areal_b200.trainer.rl_trainer import PPOTrainer
    from areal_b200.workflow.rlvr import RLVRWorkflow

    srv = _Server(0)
    try:
        monkeypatch.setenv("AREAL_LLM_SERVER_ADDRS", srv.addr)
        cfg = GRPOConfig(experiment_name="ext", trial_name="t")
        cfg.cluster.fileroot = str(tmp_path)
        cfg.train_dataset.batch_size = 4
        cfg.train_dataset.shuffle = False
        cfg.gconfig = GenerationHyperparameters(n_samples=2, max_new_tokens=8, temperature=1.0, ignore_eos=True)
        cfg.actor = PPOActorConfig(backend="fsdp:d1", model_preset="tiny-qwen2", init_from_scratch=True,
                                   optimizer=OptimizerConfig(lr=1e-3, warmup_steps_proportion=0.0),
                                   mb_spec=MicroBatchSpec(max_tokens_per_mb=1024), ppo_n_minibatches=1,
                                   reward_norm=NormConfig(mean_level="group", std_level="group", group_size=2),
                                   kl_ctl=0.0, use_decoupled_loss=True, recompute_logprob=True)
        cfg.rollout = InferenceEngineConfig(backend="native:d1", max_head_offpolicyness=0, max_concurrent_rollouts=16,
                                            setup_timeout=30.0, request_timeout=60.0)
        _propagate_names(cfg)
        g = torch.Generator().manual_seed(0)
        ds = [dict(input_ids=torch.randint(0, 1024, (12,), generator=g).tolist()) for _ in range(16)]
        before = srv.engine.flat.flat.clone()
        seen = []
        with PPOTrainer(cfg, ds) as tr:
            assert tr.external_rollout and tr.rollout is None
            tr.train(workflow=RLVRWorkflow, workflow_kwargs=dict(
                reward_fn=lambda p, c, pi, ci, **kw: float(sum(ci) % 2), gconfig=cfg.gconfig, reward_in_process=True),
                max_steps=2, step_callback=lambda s, st: seen.append(st))
            trained = tr.actor_engine.flat.flat.clone()
        assert len(seen) == 2 and all(s["step/trained_tokens"] > 0 for s in seen)
        assert srv.engine.get_version() == 2
        n = min(trained.numel(), srv.engine.flat.flat.numel())
        assert torch.allclose(srv.engine.flat.flat[:n].float(), trained[:n].float(), atol=1e-6)
        assert not torch.equal(srv.engine.flat.flat, before)
    finally:
        srv.stop()


def test_vllm_server_control_routes_against_a_stub_engine_client(tmp_path):
    """The routes ``VLLMBackend`` calls, mounted on an app whose ``engine_client`` is a stub with vLLM's
    asynchronous interface: pause aborts, an update reloads every worker from the path and drops the prefix
    cache (pausing around it when the caller did not), versions are kept, the collective routes say 501."""
    from fastapi import FastAPI
    from fastapi.testclient import TestClient

    from areal_b200.api.io_struct import WeightUpdateMeta
    from areal_b200.engine.vllm_server import attach_areal_routes

    class StubEngine:
        def __init__(self):
            self.calls = []

        async def pause_generation(self, *, mode="abort", wait_for_inflight_requests=False, clear_cache=True):
            self.calls.append(("pause", mode))

        async def resume_generation(self):
            self.calls.append(("resume",))

        async def collective_rpc(self, method, timeout=None, args=(), kwargs=None):
            self.calls.append(("rpc", method, dict(kwargs or {})))

        async def reset_prefix_cache(self):
            self.calls.append(("reset_prefix_cache",))

    app = FastAPI()
    c = TestClient(attach_areal_routes(app))
    assert c.post("/areal_pause_generation", json={}).status_code == 503          # no engine yet
    eng = app.state.engine_client = StubEngine()
    be = VLLMBackend()
    # the sequence the remote engine issues for a disk update: pause, update, resume
    assert c.post(be.pause().endpoint, json=be.pause().payload).json()["paused"] is True
    up = be.update_from_disk(WeightUpdateMeta(type="disk", path=str(tmp_path / "v3")))
    r = c.post(up.endpoint, json=dict(up.payload, version=3)).json()
    assert r["success"] and r["model_path"].endswith("v3")
    assert c.post(be.resume().endpoint, json={}).json()["paused"] is False
    assert eng.calls == [("pause", "abort"), ("rpc", "reload_weights", {"weights_path": str(tmp_path / "v3")}),
                         ("reset_prefix_cache",), ("resume",)]
    assert c.post("/areal_get_version", json={}).json()["version"] == 3
    # an update without a pause before it pauses and resumes by itself
    eng.calls.clear()
    c.post("/areal_update_weights", json={"model_path": "/ckpt/v4"})
    assert [x[0] for x in eng.calls] == ["pause", "rpc", "reset_prefix_cache", "resume"]
    assert c.post("/areal_update_weights", json={}).status_code == 400
    assert c.post("/areal_set_version", json={"version": 9}).json()["version"] == 9
    for route in ("/areal_init_weights_update_group", "/areal_set_update_weight_meta", "/areal_update_weights_xccl"):
        assert c.post(route, json={}).status_code == 501
    assert c.post("/areal_update_weights_lora", json={"lora_name": "a"}).status_code == 400
