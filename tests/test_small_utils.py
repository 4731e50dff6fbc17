"""Small utilities: parameter estimates, proximal log-prob approximations, address helpers, optional logger
backends, dynamic imports, token-balanced batch splitting."""
import dataclasses
import os
import sys
import types

import pytest
import torch

from areal_b200.models.config import PRESETS


@pytest.mark.parametrize("preset", ["tiny-qwen2", "tiny-qwen2-4l", "tiny-qwen3-moe", "tiny-qwen2_5-vl"])
def test_num_params_matches_the_built_model(preset):
    from areal_b200.models.qwen import build_model

    cfg = PRESETS[preset]
    model = build_model(cfg, dtype=torch.float32, seed=0)
    counted = sum(p.numel() for p in model.parameters())
    assert cfg.num_params() == counted
    critic = dataclasses.replace(PRESETS["tiny-qwen2"], is_critic=True)
    assert critic.num_params() == sum(p.numel() for p in build_model(critic, dtype=torch.float32, seed=0).parameters())


def test_full_size_presets_have_the_published_sizes():
    assert abs(PRESETS["qwen3-1.7b"].num_params() / 1e9 - 1.72) < 0.05
    assert abs(PRESETS["qwen3-8b"].num_params() / 1e9 - 8.19) < 0.1
    assert abs(PRESETS["qwen2.5-7b"].num_params() / 1e9 - 7.62) < 0.05
    assert abs(PRESETS["qwen3-30b-a3b"].num_params() / 1e9 - 30.5) < 0.5
    assert abs(PRESETS["llama3.1-8b"].num_params() / 1e9 - 8.03) < 0.05


def test_proximal_logprob_approximations_interpolate_by_version():
    from areal_b200.utils.functional import compute_prox_logp_approximations

    old = torch.log(torch.tensor([0.5, 0.2, 0.2, 0.2, 0.1]))
    cur = torch.log(torch.tensor([0.5, 0.4, 0.4, 0.4, 0.3]))
    versions = torch.tensor([-1, 5, 3, 4, 0])             # prompt token; fresh; 2 back; 1 back; very stale
    out = compute_prox_logp_approximations(old, cur, versions, current_version=5)
    alpha = torch.tensor([0.0, 0.0, 0.5, 0.0, 0.8])        # (v_prox - v_b) / (v_theta - v_b) with v_prox = 4
    assert torch.allclose(out["loglinear"], old + alpha * (cur - old), atol=1e-6)
    assert torch.allclose(out["linear"].exp(), (1 - alpha) * old.exp() + alpha * cur.exp(), atol=1e-6)
    assert torch.equal(out["rollout"], old)
    # both interpolations stay between the behaviour and the current log-prob, the geometric one below the arithmetic
    lo, hi = torch.minimum(old, cur), torch.maximum(old, cur)
    for k in ("loglinear", "linear"):
        assert bool(((out[k] >= lo - 1e-6) & (out[k] <= hi + 1e-6)).all())
    assert bool((out["loglinear"] <= out["linear"] + 1e-6).all())
    only = compute_prox_logp_approximations(old, cur, versions, 5, method="linear")
    assert set(only) == {"linear"}
    # every token produced by the current weights: the proximal policy is the behaviour policy
    same = compute_prox_logp_approximations(old, cur, torch.full((5,), 7), 7)
    assert torch.allclose(same["loglinear"], old)


def test_address_helpers_handle_ipv6():
    from areal_b200.utils.network import find_free_ports, format_addr, format_url, is_ipv6, split_addr

    assert format_addr("10.0.0.1", 80) == "10.0.0.1:80" and format_addr("fe80::1", 80) == "[fe80::1]:80"
    assert format_addr("[::1]", 8000) == "[::1]:8000"
    assert split_addr("[fe80::1]:80") == ("fe80::1", 80) and split_addr("host:9") == ("host", 9)
    assert split_addr("http://[::1]:8000/v1") == ("::1", 8000)
    assert format_url("::1", 8000, path="/health") == "http://[::1]:8000/health"
    assert is_ipv6("::1") and is_ipv6("[fe80::1%eth0]") and not is_ipv6("127.0.0.1") and not is_ipv6("host")
    for bad in ("fe80::1:80", "[::1]", "nohostport"):
        with pytest.raises(ValueError):
            split_addr(bad)
    ports = find_free_ports(3)
    assert len(set(ports)) == 3 and all(1024 <= p <= 65535 for p in ports)


def test_optional_logger_backends_receive_every_commit(tmp_path, monkeypatch):
    from areal_b200.api.cli_args import StatsLoggerConfig
    from areal_b200.utils.stats_logger import StatsLogger

    calls = {"swanlab": [], "trackio": []}

    def fake(name):
        m = types.ModuleType(name)
        m.init = lambda **kw: calls[name].append(("init", kw))
        m.log = lambda item, step=None: calls[name].append(("log", step, dict(item)))
        m.finish = lambda: calls[name].append(("finish",))
        m.login = lambda key: calls[name].append(("login", key))
        return m

    monkeypatch.setitem(sys.modules, "swanlab", fake("swanlab"))
    monkeypatch.setitem(sys.modules, "trackio", fake("trackio"))
    cfg = StatsLoggerConfig(experiment_name="exp", trial_name="t", fileroot=str(tmp_path))
    cfg.swanlab.mode, cfg.swanlab.api_key = "local", "k"
    cfg.trackio.mode, cfg.trackio.space_id = "online", "me/space"
    lg = StatsLogger(cfg)
    lg.commit(0, 0, 0, {"loss": 1.5})
    lg.commit(0, 1, 1, [{"loss": 1.0}, {"loss": 0.5}])
    lg.close()
    assert calls["swanlab"][0] == ("login", "k") and calls["swanlab"][1][1]["project"] == "exp"
    assert calls["trackio"][0][1] == {"project": "exp", "name": "t", "space_id": "me/space"}
    for name in calls:
        logs = [c for c in calls[name] if c[0] == "log"]
        assert [c[1] for c in logs] == [0, 2, 3] and logs[-1][2] == {"loss": 0.5}
        assert calls[name][-1] == ("finish",)
    # a backend that cannot start is skipped, the run goes on
    broken = types.ModuleType("swanlab")
    broken.init = lambda **kw: (_ for _ in ()).throw(RuntimeError("no server"))
    monkeypatch.setitem(sys.modules, "swanlab", broken)
    lg2 = StatsLogger(cfg)
    lg2.commit(0, 0, 0, {"loss": 1.0})
    lg2.close()


def test_import_from_string_forms(tmp_path):
    from areal_b200.utils.dynamic_import import import_from_string

    assert import_from_string("areal_b200.reward.gsm8k.gsm8k_reward_fn").__name__ == "gsm8k_reward_fn"
    assert import_from_string("areal_b200.workflow.rlvr:RLVRWorkflow").__name__ == "RLVRWorkflow"
    assert import_from_string("os.path:join") is __import__("os").path.join
    assert import_from_string("areal_b200.utils.network").__name__ == "areal_b200.utils.network"
    script = tmp_path / "user_code.py"
    script.write_text("class Agent:\n    tag = 7\n\ndef reward(*a, **k):\n    return 1.0\n")
    assert import_from_string(f"{script}:Agent.tag") == 7
    assert import_from_string(f"{script}:reward")() == 1.0
    assert import_from_string(f"{script}:Agent") is import_from_string(f"{script}:Agent")   # loaded once
    for bad in ("areal_b200.reward.gsm8k.nope", "no_such_pkg_xyz.f", ""):
        with pytest.raises((ImportError, ValueError, AttributeError)):
            import_from_string(bad)


def test_batches_are_split_by_tokens_with_groups_kept_together():
    from areal_b200.infra.dist_rollout import split_batch_by_tokens

    lens = [10, 12, 90, 95, 50, 48, 30, 33]               # 4 groups of 2
    B, L = len(lens), 100
    mask = torch.zeros(B, L, dtype=torch.bool)
    for i, n in enumerate(lens):
        mask[i, :n] = True
    batch = {"attention_mask": mask, "input_ids": torch.arange(B)[:, None].expand(B, L).clone(),
             "rewards": torch.arange(B, dtype=torch.float32), "meta": "kept"}
    parts = split_batch_by_tokens(batch, 2, group_size=2)
    assert len(parts) == 2 and all(p["meta"] == "kept" for p in parts)
    rows = [p["rewards"].long().tolist() for p in parts]
    assert sorted(sum(rows, [])) == list(range(B)) and all(len(r) == 4 for r in rows)
    for r in rows:                                         # groups (2k, 2k+1) stay together
        assert all((i ^ 1) in r for i in r)
    tokens = [int(p["attention_mask"].sum()) for p in parts]
    assert sorted(tokens) == [161, 207]                    # 98 + 63 and 185 + 22: the heavy group pairs with the light one
    assert split_batch_by_tokens(batch, 1)[0] is batch


def test_engine_api_conveniences(tmp_path):
    """``initialized``, device statistics, perf-tracer hooks and rollout forwarded through the connected engine."""
    from areal_b200.api.cli_args import (InferenceEngineConfig, NativeRolloutConfig, OptimizerConfig, PerfTracerConfig,
                                         TrainEngineConfig)
    from areal_b200.api.io_struct import DeviceRuntimeInfo, WeightUpdateMeta
    from areal_b200.engine.rollout_engine import NativeRolloutEngine
    from areal_b200.engine.train_engine import B200TrainEngine
    from areal_b200.infra.workflow_executor import WorkflowExecutor
    from areal_b200.workflow.rlvr import RLVRWorkflow

    info = DeviceRuntimeInfo.get_current("MB")
    assert info.unit == "MB" and "memory [MB]" in info.log("step 0")
    with pytest.raises(ValueError):
        DeviceRuntimeInfo.get_current("TB")
    eng = B200TrainEngine(TrainEngineConfig(experiment_name="e", trial_name="t", path="", init_from_scratch=True,
                                            dtype="float32", model_preset="tiny-qwen2", optimizer=OptimizerConfig()))
    assert not eng.initialized
    eng.create_process_group()
    eng.initialize(seed=0)
    assert eng.initialized and eng.get_device_stats().unit == "GB"
    eng.start_memory_profile()
    eng.stop_memory_profile(str(tmp_path / "mem"))            # no CUDA here: both are no-ops
    with pytest.raises(RuntimeError, match="connect_engine"):
        eng.rollout_batch([{"input_ids": [1, 2, 3]}], workflow=None)
    rcfg = InferenceEngineConfig(experiment_name="e", trial_name="t", backend="native:d1", max_concurrent_rollouts=8,
                                 consumer_batch_size=2,
                                 native=NativeRolloutConfig(model_preset="tiny-qwen2", context_length=64, max_num_seqs=8,
                                                            max_num_batched_tokens=256, num_kv_blocks=32, seed=0,
                                                            cuda_graph=False))
    ro = NativeRolloutEngine(rcfg)
    assert not ro.initialized
    with pytest.raises(RuntimeError):
        ro.workflow_executor
    ro.initialize(device="cpu")
    try:
        assert ro.initialized and isinstance(ro.workflow_executor, WorkflowExecutor)
        eng.connect_engine(ro, WeightUpdateMeta(type="colocated") if hasattr(WeightUpdateMeta, "type") else None)
        from areal_b200.api.cli_args import GenerationHyperparameters

        g = GenerationHyperparameters(max_new_tokens=4, greedy=True, ignore_eos=True)
        wf = RLVRWorkflow(reward_fn=lambda *a, **k: 1.0, gconfig=g, reward_in_process=True)
        batch = eng.rollout_batch([{"input_ids": [5, 6, 7]}, {"input_ids": [8, 9]}], workflow=wf)
        assert batch["input_ids"].shape[0] == 2 and batch["rewards"].tolist() == [1.0, 1.0]
        eng.config_perf_tracer(PerfTracerConfig(experiment_name="e", trial_name="t", fileroot=str(tmp_path), enabled=True),
                               rank=0, role="actor")
        eng.save_perf_tracer(step=0, force=True)
        ro.save_perf_tracer(force=True)
    finally:
        from areal_b200.utils import perf_tracer

        perf_tracer.configure(None)
        ro.destroy()
        eng.destroy()


def test_container_and_padding_helpers():
    from areal_b200.utils import data as D

    items = [{"a": 1, "b": "x"}, {"a": 2, "b": "y"}]
    d = D.list_of_dict2dict_of_list(items)
    assert d == {"a": [1, 2], "b": ["x", "y"]} and D.dict_of_list2list_of_dict(d) == items
    with pytest.raises(ValueError):
        D.list_of_dict2dict_of_list([{"a": 1}, {"b": 2}])
    with pytest.raises(ValueError):
        D.dict_of_list2list_of_dict({"a": [1], "b": [1, 2]})
    assert D.dict_map(lambda v: v * 2, {"a": 1}) == {"a": 2}
    moved = D.tensor_container_to({"x": torch.ones(2), "l": [torch.zeros(1), "s"], "n": 3}, torch.float64)
    assert moved["x"].dtype == torch.float64 and moved["l"][0].dtype == torch.float64 and moved["l"][1] == "s"
    st = D.pad_and_stack_tensors_along_first_dim([torch.ones(2, 3), torch.ones(4, 3)], pad_value=-1)
    assert st.shape == (2, 4, 3) and (st[0, 2:] == -1).all()
    mask = torch.tensor([[1, 1, 1, 0], [1, 0, 0, 0], [1, 1, 0, 0]])
    x = torch.arange(12.0).reshape(3, 4, 1) + 1
    packed, idx, cu, mx = D.unpad_input(x, mask)
    assert packed.squeeze(-1).tolist() == [1, 2, 3, 5, 9, 10] and cu.tolist() == [0, 3, 4, 6] and mx == 3
    back = D.pad_input(packed, idx, 3, 4)
    assert torch.equal(back, x * mask[..., None])
    seqs = D.unpack_sequence(packed, cu)
    assert [s.shape[0] for s in seqs] == [3, 1, 2] and [s.shape[0] for s in D.unpack_sequence(packed, lens=[2, 4])] == [2, 4]
    batch = {"input_ids": torch.arange(10).reshape(5, 2), "attention_mask": torch.ones(5, 2, dtype=torch.bool),
             "images": list("abcde"), "meta": "m"}
    parts = D.split_batch(batch, 3)
    assert [p["input_ids"].shape[0] for p in parts] == [2, 2, 1] and parts[2]["images"] == ["e"] and parts[0]["meta"] == "m"
    whole = D.concat_batch([{k: v for k, v in p.items() if torch.is_tensor(v)} for p in parts])
    assert torch.equal(whole["input_ids"], batch["input_ids"])
    with pytest.raises(ValueError):
        D.split_batch(batch, 6)
    dummy = D.make_dummy_eval_item({"input_ids": torch.ones(1, 7, dtype=torch.long), "attention_mask": torch.ones(1, 7, dtype=torch.bool),
                                    "loss_mask": torch.ones(1, 7, dtype=torch.int32), "rewards": torch.ones(1), "images": ["i"]})
    assert dummy["input_ids"].shape == (1, 1) and bool(dummy["attention_mask"].all()) and int(dummy["loss_mask"].sum()) == 0
    assert dummy["images"] == [None] and D.broadcast_tensor(torch.ones(2)).tolist() == [1.0, 1.0]


def test_more_small_helpers(tmp_path):
    from areal_b200.api.cli_args import RecoverConfig, conf_as_dict, get_py_cmd
    from areal_b200.api.io_struct import StepInfo, detect_image_mime, get_versioned_lora_name
    from areal_b200.utils import network as N
    from areal_b200.utils.recover import InValidRecoverInfo, InvalidRecoverInfo, RecoverHandler, RecoverInfo, check_if_auto_recover

    assert N.format_hostport("::1", 5) == "[::1]:5" and N.split_hostport("[::1]:5") == ("::1", 5)
    assert N.format_host_for_url("fe80::1") == "[fe80::1]" and N.format_host_for_url("h") == "h"
    port = N.find_free_ports(1)[0]
    assert N.is_port_free(port, "127.0.0.1")
    import socket

    with socket.socket() as s:
        s.bind(("127.0.0.1", port))
        s.listen()
        assert not N.is_port_free(port, "127.0.0.1")
    assert N.get_loopback_ip() == "127.0.0.1" and N.get_loopback_ip(True) in ("::1", "127.0.0.1") and N.gethostname()
    assert get_versioned_lora_name("ad", 3) == "ad-v3"
    import base64

    assert detect_image_mime(base64.b64encode(b"\x89PNG\r\n\x1a\n0000").decode()) == "image/png"
    assert detect_image_mime(base64.b64encode(b"\xff\xd8\xff\xe0data").decode()) == "image/jpeg"
    assert detect_image_mime(base64.b64encode(b"GIF89a....").decode()) == "image/gif"
    assert detect_image_mime("????") == "image/jpeg"
    assert get_py_cmd("pkg.mod", {"model_path": "/m", "tp": 2, "trust": True, "skip": False, "none": None, "ids": [1, 2],
                                  "empty": []}) == ["python3", "-m", "pkg.mod", "--model-path", "/m", "--tp", "2",
                                                    "--trust", "--ids", "1", "2"]
    cfg = RecoverConfig(experiment_name="e", trial_name="t", fileroot=str(tmp_path), mode="auto")
    assert conf_as_dict(cfg)["mode"] == "auto" and conf_as_dict({"a": 1}) == {"a": 1}
    assert InValidRecoverInfo is InvalidRecoverInfo and not check_if_auto_recover(cfg)
    root = os.path.join(RecoverHandler.recover_root(cfg), "recover_info")
    RecoverInfo(last_step_info=StepInfo(0, 1, 1, 4), checkpoint_info={"path": str(tmp_path / "missing")}).dump(root)
    assert not check_if_auto_recover(cfg)                       # the checkpoint it names is gone
    os.makedirs(tmp_path / "missing")
    assert check_if_auto_recover(cfg)


def test_stateful_loader_resumes_mid_epoch_and_splits_evaluation_exactly():
    from areal_b200.utils.data import cycle_dataloader
    from areal_b200.utils.dataloader import StatefulListLoader, create_dataloader

    data = list(range(23))
    # training: both ranks get the same number of batches, disjoint samples, a new order every epoch
    loaders = [StatefulListLoader(data, 3, shuffle=True, seed=7, rank=r, world=2) for r in range(2)]
    assert len(loaders[0]) == len(loaders[1]) == 3                      # 22 usable samples -> 11 per rank -> 3 batches
    e0 = [list(ld) for ld in loaders]
    assert all(len(b) == 3 for ep in e0 for b in ep) and len(e0[0]) == len(e0[1]) == 3
    seen = [x for ep in e0 for b in ep for x in b]
    assert len(set(seen)) == len(seen) == 18
    e1 = list(loaders[0])
    assert loaders[0].epoch == 2 and e1 != e0[0]
    # a checkpoint in the middle of an epoch continues with the next batch of the same permutation
    a = StatefulListLoader(data, 2, shuffle=True, seed=1)
    it = iter(a)
    first = [next(it), next(it)]
    state = a.state_dict()
    assert state == {"epoch": 0, "position": 2}
    rest = list(it)
    b = StatefulListLoader(data, 2, shuffle=True, seed=1)
    b.load_state_dict(state)
    assert list(b) == rest and b.epoch == 1 and b.position == 0
    # the endless iterator keeps a restored loader's place and moves through epochs
    c = StatefulListLoader(data, 2, shuffle=True, seed=1)
    c.load_state_dict(state)
    cyc = cycle_dataloader(c)
    got = [next(cyc) for _ in range(len(rest) + 2)]
    fresh = StatefulListLoader(data, 2, shuffle=True, seed=1)
    fresh.set_epoch(1)
    assert got[: len(rest)] == rest and got[len(rest):] == [next(i) for i in [iter(fresh)] * 2]
    assert first[0] not in rest
    # evaluation: every sample exactly once, ranks differ by at most one, nothing padded
    ev = [StatefulListLoader(data, 4, shuffle=False, rank=r, world=3, drop_last=False) for r in range(3)]
    per_rank = [[x for bt in ld for x in bt] for ld in ev]
    assert sorted(x for pr in per_rank for x in pr) == data and {len(pr) for pr in per_rank} == {7, 8}
    assert [len(ld) for ld in ev] == [2, 2, 2]

    class ValidDatasetConfig:
        batch_size, shuffle, drop_last = 6, False, True

    class TrainDatasetConfig:
        batch_size, shuffle, drop_last = 6, True, True

    v = create_dataloader(data, 1, 3, ValidDatasetConfig())
    assert (v.batch_size, v.drop_last, v.shuffle) == (2, False, False)
    t = create_dataloader(data, 0, 3, TrainDatasetConfig(), collate_fn=lambda items: sum(items))
    assert t.drop_last and isinstance(next(iter(t)), int)
    with pytest.raises(ValueError):
        create_dataloader(data, 0, 4, TrainDatasetConfig())


def test_tiny_utility_modules(tmp_path, monkeypatch):
    from areal_b200.utils import constants, environ, errors, fs, image, pkg_version, printing, wrapper
    from areal_b200.utils.math import align, ceil_div

    assert ceil_div(7, 2) == 4 and ceil_div(8, 2) == 4 and align(17, 16) == 32 and align(32, 16) == 32
    e = errors.EngineError("update", "timeout", "no ack")
    assert "sub_error: timeout" in str(e) and isinstance(errors._Structured.from_dict(e.to_dict()), errors.EngineError)
    assert isinstance(errors.FrameworkError.from_dict(errors.FrameworkError("a", "b", "c").to_dict()), errors.FrameworkError)
    monkeypatch.setenv("X_FLAG", "TRUE")
    assert environ.get_bool_env_var("X_FLAG") and not environ.get_bool_env_var("X_MISSING")
    monkeypatch.setenv("X_FLAG", "maybe")
    assert not environ.get_bool_env_var("X_FLAG")
    monkeypatch.delenv("RANK", raising=False)
    monkeypatch.delenv("AREAL_SPMD_MODE", raising=False)
    assert environ.is_single_controller() and not environ.is_in_ci()
    monkeypatch.setenv("RANK", "0")
    assert not environ.is_single_controller()
    table = printing.tabulate_stats({f"k{i}": float(i) for i in range(5)}, col=2)
    assert "k0" in table and "k4" in table and "4.0000e+00" in table and printing.tabulate_stats({}) == "(no stats)"
    from PIL import Image

    a, b = Image.new("RGB", (4, 2), (255, 0, 0)), Image.new("RGB", (2, 6), (0, 255, 0))
    enc = image.image2base64([a, b])
    assert len(enc) == 2 and image.base642image("data:image/png;base64," + enc[0]).size == (4, 2)
    from areal_b200.api.io_struct import detect_image_mime

    assert detect_image_mime(enc[0]) == "image/png"
    padded = image.pad_images_batch_to_max_size([a, b])
    assert [p.size for p in padded] == [(4, 6), (4, 6)] and padded[0].getpixel((0, 0)) == (0, 0, 0)
    assert padded[0].getpixel((0, 2)) == (255, 0, 0)

    class Engine:
        @wrapper.wrapable()
        def step(self, x):
            return x + 1

        @wrapper.wrapable("renamed")
        def other(self):
            return "o"

        def hidden(self):
            return None

    class Proxy:
        pass

    calls = []

    def via_rpc(*args, **kwargs):
        calls.append(wrapper.wrap_get_method_name(kwargs))
        fn = wrapper.wrap_get_method(kwargs)
        return fn(*args, **wrapper.wrap_remove_meta(kwargs))

    p = Proxy()
    assert sorted(wrapper.wrap(p, Engine(), via_rpc)) == ["renamed", "step"]
    assert p.step(1) == 2 and p.renamed() == "o" and calls == ["step", "renamed"] and not hasattr(p, "hidden")
    q = Proxy()
    wrapper.wrap(q, Engine())
    assert q.step(x=4) == 5
    assert pkg_version.is_available("torch") and not pkg_version.is_available("surely_not_a_package_xyz")
    assert pkg_version.compare_versions("2.11.0+cu128", "2.9") == 1 and pkg_version.compare_versions("1.2.0rc1", "1.2.0") == -1
    assert pkg_version.compare_versions("v0.5", "0.5.0") == 0 and pkg_version.compare_versions("1.0.post1", "1.0") == 1
    assert pkg_version.is_version_greater_or_equal("torch", "2.0") and pkg_version.is_version_less("torch", "99")
    with pytest.raises(ValueError):
        pkg_version.compare_versions("abc", "1.0")
    assert os.path.isdir(fs.get_user_tmp())
    fs.validate_shared_path(str(tmp_path / "new" / "dir"), "fileroot", n_nodes=2)   # an ancestor exists and is writable
    with pytest.raises(ValueError):
        fs.validate_shared_path("", "fileroot")
    assert fs.is_network_fs(str(tmp_path)) in (True, False, None)
    assert constants.DEFAULT_VECTORIZED_ALIGNMENT_BYTES == 16 and "recompute" in constants.PROX_LOGP_METHODS_ALL


def test_partition_schedule_and_seed_helpers():
    import numpy as np

    from areal_b200.utils import names, seqpack, timeutil
    from areal_b200.utils.seeding import Shuffler

    assert seqpack.get_allocate_fn("ffd") is seqpack.ffd_allocate and seqpack.get_allocate_fn("kk") is seqpack.kk_allocate
    with pytest.raises(ValueError):
        seqpack.get_allocate_fn("best")
    parts = seqpack.min_abs_diff_partition([5, 1, 1, 1, 5, 1, 1, 5], 3)
    assert parts[0][0] == 0 and parts[-1][1] == 8 and len(parts) == 3
    sums = [sum([5, 1, 1, 1, 5, 1, 1, 5][a:b]) for a, b in parts]
    assert max(sums) == 7                                          # [5,1,1] [1,5,1] [1,5] or as good
    with pytest.raises(ValueError):
        seqpack.min_abs_diff_partition([1, 2], 3)
    with pytest.raises(ValueError):
        seqpack.min_abs_diff_partition(np.ones((2, 2)), 1)
    lens = [100, 90, 10, 10, 50, 50, 40, 60]
    perm, diff = seqpack.reorder_to_balanced_batches(lens, 2)
    assert sorted(perm.tolist()) == list(range(8))
    loads = [sum(lens[i] for i in perm[j:j + 2]) for j in range(0, 8, 2)]
    assert max(loads) - min(loads) == diff and diff <= 10 and loads == sorted(loads, reverse=True)
    assert seqpack.flat2d([[1, 2], [3]]) == [1, 2, 3]
    lin = timeutil.LinearScheduler(1.0, 10, end_value=0.0)
    assert lin.get(0) == 1.0 and abs(lin.get(5) - 0.5) < 1e-12 and lin.final_value == 0.0
    cos = timeutil.CosineDecayScheduler(1.0, 10, end_value=0.2)
    assert cos.get(0) == 1.0 and abs(cos.get(5) - 0.6) < 1e-12 and abs(cos.get(10) - 0.2) < 1e-12
    assert abs(timeutil.ExponentialScheduler(2.0, 4, decay=0.5).get(3) - 0.25) < 1e-12
    ch = timeutil.ChainedScheduler([timeutil.ConstantScheduler(1.0, 3), lin])
    assert ch.total_iters == 13 and ch.get(2) == 1.0 and abs(ch.get(8) - 0.5) < 1e-12 and ch.final_value == 0.0
    with pytest.raises(ValueError):
        timeutil.ChainedScheduler([lin, timeutil.ConstantScheduler(1.0, 3)])   # 0.0 does not meet 1.0
    with pytest.raises(ValueError):
        lin.get(11)
    a, b = Shuffler("k"), Shuffler("k")
    sa = [a.next_shuffle() for _ in range(3)]
    assert sa == [b.next_shuffle() for _ in range(3)] and len(set(sa)) == 3 and Shuffler("other").next_shuffle() != sa[0]
    c = Shuffler("k")
    c.load_state_dict({"key": "k", "cnt": 2})
    assert c.next_shuffle() == sa[2]
    assert names.trial_registry("e", "t").endswith("/e/t") and names.trial_registry("e", "t").startswith(names.registry_root())
    assert names.worker_discovery("e", "t", "rollout") == names.workers("e", "t", "rollout")
    assert names.worker_discovery("e", "t", "rollout", 3) == names.worker("e", "t", "rollout", 3)


def test_trajectories_are_rebalanced_over_data_parallel_ranks():
    import subprocess
    import sys

    from tests.conftest import free_port

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(free_port()), os.path.join(root, "tests", "torchrun", "run_redistribute.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "OK" in r.stdout, r.stdout[-1500:] + r.stderr[-2500:]
    # one rank: nothing to do
    from areal_b200.infra.dist_rollout import DistRolloutCoordinator, redistribute_trajectories

    b = {"attention_mask": torch.ones(3, 4, dtype=torch.bool), "x": torch.arange(3)}
    out = redistribute_trajectories(b)
    assert out.data is b and out.group_indices == [[0, 1, 2]]
    assert redistribute_trajectories(None).data == {}

    class Eng:
        data_parallel_world_size, data_parallel_group, context_and_model_parallel_group = 1, None, None

        def is_data_parallel_head(self):
            return True

        def current_data_parallel_head(self):
            return 0

    class Ro:
        def rollout_batch(self, data, workflow=None, workflow_kwargs=None, group_size=1):
            return dict(b, n=len(data))

        def prepare_batch(self, dl, workflow=None, workflow_kwargs=None, should_accept_fn=None, group_size=1, dynamic_bs=False):
            return dict(b, dyn=dynamic_bs)

    co = DistRolloutCoordinator(Ro(), Eng())
    assert co.rollout_batch([1, 2])["n"] == 2 and co.prepare_batch(None, dynamic_bs=True)["dyn"] is True


def test_reference_named_entry_points_exist_and_work():
    from areal_b200.reward import MathVerifyWorker, get_math_verify_worker
    from areal_b200.trainer.ppo.actor import PPOActorController, PPOActorControllerV2, compute_prox_logp_approximations
    from areal_b200.trainer.ppo.critic import PPOCriticController, PPOCriticEngine, critic_loss_fn, ppo_loss_fn
    from areal_b200.infra.controller.train_controller import TrainController
    from areal_b200.workflow.rlvr import default_data_extract_prompt_fn, default_get_input_ids, default_get_input_ids_fn

    w = get_math_verify_worker()
    assert w is get_math_verify_worker() and isinstance(w, MathVerifyWorker)
    assert w.verify("so the result is \\boxed{42}", "42") == 1.0 and w.verify("it is \\boxed{41}", "42") == 0.0
    assert w.verify(None, "42") == 0.0 and w.verify("\\boxed{\\frac{1}{2}}", "0.5") == 1.0
    assert issubclass(PPOActorController, TrainController) and PPOActorControllerV2 is PPOActorController
    assert issubclass(PPOCriticController, TrainController) and ppo_loss_fn is critic_loss_fn and callable(compute_prox_logp_approximations)
    assert hasattr(PPOCriticEngine, "compute_values") and default_get_input_ids_fn is default_get_input_ids
    assert default_data_extract_prompt_fn({"messages": [{"role": "user", "content": "q"}]})[0]["content"] == "q"
    assert default_data_extract_prompt_fn({"input_ids": [1, 2]}) == [1, 2]


def test_http_helper_passes_headers(monkeypatch):
    """The gateway-side engines authenticate with a bearer header: the retrying helper has to carry it."""
    import requests

    from areal_b200.infra.utils import http

    seen = {}

    class R:
        status_code = 200
        text = "{}"

        def json(self):
            return {}

    def fake(method, url, **kw):
        seen.update(kw, method=method, url=url)
        return R()

    monkeypatch.setattr(requests, "request", fake)
    http.request_with_retry("POST", "http://x/y", json={"a": 1}, headers={"Authorization": "Bearer t"}, max_retries=0)
    assert seen["headers"] == {"Authorization": "Bearer t"} and seen["json"] == {"a": 1}
    http.request_with_retry("GET", "http://x/y", max_retries=0)
    assert seen["headers"] is None


def test_sdpa_general_attention_path_matches_the_reference():
    """The path long sequences take when the head width has no tcgen05 kernel: same values and gradients as the
    fp32 reference, with grouped-query heads and several packed sequences (one of them empty)."""
    import torch

    from areal_b200.ops.attention import attention_ref, attention_sdpa

    g = torch.Generator().manual_seed(0)
    cu = [0, 17, 17, 60, 64]
    q = torch.randn(64, 6, 48, generator=g, requires_grad=True)
    k = torch.randn(64, 2, 48, generator=g, requires_grad=True)
    v = torch.randn(64, 2, 48, generator=g, requires_grad=True)
    want = attention_ref(q, k, v, cu, 0.11)
    got = attention_sdpa(q, k, v, cu, 0.11)
    assert torch.allclose(got, want, atol=1e-5)
    w = torch.randn(64, 6, 48, generator=g)
    gw = torch.autograd.grad((want * w).sum(), (q, k, v))
    gg = torch.autograd.grad((got * w).sum(), (q, k, v))
    assert all(torch.allclose(a, b, atol=1e-5) for a, b in zip(gw, gg))
