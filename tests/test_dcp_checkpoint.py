"""torch.distributed.checkpoint format of the train engine: resharding across data-parallel sizes and
across parallel layouts, resume under tensor / pipeline / expert parallelism, background writes, and reading a
checkpoint in the layout the reference's FSDP engine writes (areal/engine/fsdp_engine.py:1668-1693)."""
import os
import subprocess
import sys

import pytest

from tests.conftest import free_port
import torch

from areal_b200.utils.dcp_state import checkpoint_keys, flat_range_boxes, load_full_tensors

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
WORKER = os.path.join(ROOT, "tests", "torchrun", "run_dcp.py")


def _run(n, port, args):
    env = {k: v for k, v in os.environ.items() if k not in ("RANK", "WORLD_SIZE", "LOCAL_RANK")}
    if n == 1:
        cmd = [sys.executable, WORKER] + args
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
               "--master-addr", "127.0.0.1", "--master-port", str(free_port()), WORKER] + args
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "OK" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]
    return [float(x) for x in r.stdout.strip().splitlines()[-1].split()[1:]]


def _tensors(path):
    out = load_full_tensors(path, "dcp.model.")
    out.update({"optim." + k: v for k, v in load_full_tensors(path, "dcp.optim.state.").items()})
    return out


def _assert_same(a, b, exact=True, tol=0.0):
    assert set(a) == set(b), sorted(set(a) ^ set(b))[:6]
    for k in a:
        if exact:
            assert torch.equal(a[k], b[k]), k
        else:
            err = (a[k].double() - b[k].double()).abs().max().item()
            # Adam steps of size lr = 2e-3 amplify reduction-order noise of tiny gradients: allow lr * 1e-3
            assert err <= tol * (a[k].abs().max().item() + 1e-8) + 2e-6, (k, err)


def test_flat_range_boxes_tile_the_range():
    shape = (3, 4, 5)
    n = 60
    ref = torch.arange(n).view(shape)
    for a in range(0, n, 7):
        for b in range(a, n + 1, 5):
            got = torch.full(shape, -1)
            total = 0
            for off, sz, start in flat_range_boxes(shape, a, b):
                sl = tuple(slice(o, o + s) for o, s in zip(off, sz))
                m = 1
                for s in sz:
                    m *= s
                got[sl] = torch.arange(start, start + m).view(sz)
                total += m
            assert total == b - a
            flat = got.view(-1)
            assert torch.equal(flat[a:b], ref.view(-1)[a:b]) and (flat[:a] == -1).all() and (flat[b:] == -1).all()


@pytest.mark.parametrize("resume_ws", [1, 4])
def test_save_at_two_ranks_load_at_another_size(tmp_path, resume_ws):
    """Saved at dp 2; loaded at dp 1 / dp 4: weights, master copy and Adam moments are bit-equal after the load,
    and the next step lands where the uninterrupted run did."""
    d = str(tmp_path)
    ref = _run(2, 29700 + 4 * resume_ws, ["--phase", "train", "--dir", d])
    got = _run(resume_ws, 29701 + 4 * resume_ws, ["--phase", "resume", "--dir", d])
    saved, reloaded = _tensors(os.path.join(d, "ckpt")), _tensors(os.path.join(d, "reload"))
    assert any(k.endswith(".exp_avg") for k in saved) and any(k.endswith(".master") for k in saved)
    _assert_same(saved, reloaded, exact=True)
    _assert_same(_tensors(os.path.join(d, "after")), _tensors(os.path.join(d, "resumed")), exact=False, tol=1e-4)
    assert abs(ref[0] - got[0]) < 1e-4 * abs(ref[0]) and abs(ref[2] - got[2]) < 1e-12  # loss and learning rate


@pytest.mark.parametrize("flags,one,preset", [(["--tp", "2"], [], "tiny-qwen2"),
                                              (["--pp", "2", "--n-mbs", "2"], ["--n-mbs", "2"], "tiny-qwen2"),
                                              (["--ep", "2"], [], "tiny-qwen3-moe"),
                                              (["--tp", "2", "--ep", "2"], [], "tiny-qwen3-moe"),
                                              (["--tp", "2", "--etp", "2"], [], "tiny-qwen3-moe"),
                                              (["--tp", "2", "--ep", "2"], [], "tiny-deepseek-v3"),
                                              (["--pp", "2", "--n-mbs", "2", "--lora"], ["--n-mbs", "2", "--lora"], "tiny-qwen2-4l"),
                                              (["--tp", "2", "--lora"], ["--lora"], "tiny-qwen2-4l")])
def test_resume_under_model_parallelism_and_on_one_rank(tmp_path, flags, one, preset):
    """Two steps, checkpoint, third step on two ranks under tensor / pipeline / expert parallelism. Resuming from
    the checkpoint under the same layout gives the same third step (scheduler and, under expert parallelism,
    the expert optimizer's counters included); a single process reads the same checkpoint too."""
    d = str(tmp_path)
    common = ["--dir", d, "--preset", preset]
    port = 29720 + 2 * len(flags) + (4 if preset != "tiny-qwen2" else 0) + (10 if "--tp" in flags and "--ep" in flags else 0) + (20 if "--etp" in flags else 0)
    ref = _run(2, 0, ["--phase", "train"] + common + flags)
    got = _run(2, 0, ["--phase", "resume"] + common + flags)
    _assert_same(_tensors(os.path.join(d, "ckpt")), _tensors(os.path.join(d, "reload")), exact=True)
    _assert_same(_tensors(os.path.join(d, "after")), _tensors(os.path.join(d, "resumed")), exact=False, tol=1e-5)
    assert abs(ref[0] - got[0]) < 1e-5 * abs(ref[0]) and abs(ref[2] - got[2]) < 1e-12
    got1 = _run(1, 0, ["--phase", "resume"] + common + one)
    _assert_same(_tensors(os.path.join(d, "ckpt")), _tensors(os.path.join(d, "reload")), exact=True)
    assert abs(ref[0] - got1[0]) < 1e-4 * abs(ref[0])


def test_background_write_uses_the_staged_copy(tmp_path):
    """``async_save``: the state is copied to host memory before ``save`` returns, the next optimizer step runs
    while the files are written, and the checkpoint holds the state of the moment of the call."""
    d, e = str(tmp_path / "a"), str(tmp_path / "b")
    _run(2, 29730, ["--phase", "train", "--dir", d, "--async-save"])
    _run(2, 29731, ["--phase", "train", "--dir", e])
    _assert_same(_tensors(os.path.join(d, "ckpt")), _tensors(os.path.join(e, "ckpt")), exact=True)


@pytest.mark.parametrize("flags", [["--tp", "2"], ["--pp", "2", "--n-mbs", "2"]])
def test_hf_weights_with_dcp_optimizer_state_under_model_parallelism(tmp_path, flags):
    """``weight_format="hf"`` with ``with_optim``: safetensors for the weights, a DCP sub-directory for the
    optimizer (tensor-parallel peers write disjoint shards of one tensor, not one file per rank). Under
    pipeline parallelism every stage loads its own blocks back from the shared directory, the last stage its
    copy of the tied embedding included."""
    d = str(tmp_path)
    ref = _run(2, 29740 + len(flags), ["--phase", "train", "--dir", d, "--format", "hf"] + flags)
    got = _run(2, 29745 + len(flags), ["--phase", "resume", "--dir", d, "--format", "hf"] + flags)
    keys = checkpoint_keys(os.path.join(d, "ckpt", "optimizer"))
    assert any(k.endswith("q_proj.weight.exp_avg") for k in keys) and not any(k.startswith("dcp.model.") for k in keys)
    assert abs(ref[0] - got[0]) < 1e-5 * abs(ref[0]) and abs(ref[2] - got[2]) < 1e-12


def test_reads_a_checkpoint_in_the_fsdp_engine_layout(tmp_path):
    """The reference saves ``{"dcp": {"model": <HF-named fp32 tensors>, "optim": ...}}``. Such a checkpoint
    (written here from an HF model with plain ``dcp.save``) loads into the engine: the logits match HF."""
    import torch.distributed.checkpoint as dcp
    from transformers import Qwen2Config, Qwen2ForCausalLM

    from areal_b200.api.cli_args import OptimizerConfig, TrainEngineConfig
    from areal_b200.api.io_struct import SaveLoadMeta
    from areal_b200.engine.train_engine import B200TrainEngine
    from areal_b200.models.config import PRESETS

    mc = PRESETS["tiny-qwen2"]
    hf_cfg = Qwen2Config(**{k: v for k, v in mc.to_hf_config().items() if k not in ("architectures", "model_type")})
    torch.manual_seed(0)
    hf = Qwen2ForCausalLM(hf_cfg).float().eval()
    sd = {k: v.detach().clone() for k, v in hf.state_dict().items()}
    if mc.tie_word_embeddings:
        sd.pop("lm_head.weight", None)
    path = str(tmp_path / "ref_ckpt")
    dcp.save({"dcp": {"model": sd}}, checkpoint_id=path, no_dist=True)
    eng = B200TrainEngine(TrainEngineConfig(experiment_name="t", trial_name="t", path="", init_from_scratch=True,
                                            dtype="float32", model_preset="tiny-qwen2",
                                            optimizer=OptimizerConfig(lr=1e-3)))
    eng.create_process_group()
    eng.initialize(seed=5)
    eng.load(SaveLoadMeta(path=path, weight_format="dcp", with_optim=True))
    ids = torch.randint(0, mc.vocab_size, (1, 24))
    with torch.no_grad():
        ref = hf(ids).logits[0]
        from areal_b200.ops.attention import VarlenMeta

        h = eng.model(ids[0], torch.arange(24), VarlenMeta([0, 24], torch.device("cpu")))
        got = eng.model.logits(h, out_dtype=torch.float32)
    torch.testing.assert_close(got, ref, atol=2e-4, rtol=2e-4)
    # the fp32 master copy was filled from the checkpoint's tensors
    o = eng.optimizer
    torch.testing.assert_close(o.master, eng.flat.flat[o.flat.shard_offset:o.flat.shard_offset + o.flat.shard_numel].float())


def test_recover_handler_round_trip_through_dcp(tmp_path):
    """``RecoverHandler.dump`` / ``load`` go through the DCP format and restore weights, optimizer and version."""
    from areal_b200.api.cli_args import OptimizerConfig, RecoverConfig, TrainEngineConfig
    from areal_b200.api.io_struct import FinetuneSpec, StepInfo
    from areal_b200.engine.train_engine import B200TrainEngine
    from areal_b200.utils.recover import RecoverHandler

    sys.path.insert(0, os.path.join(ROOT, "tests", "torchrun"))
    from run_dcp import batch_of, loss_fn

    def make(seed):
        e = B200TrainEngine(TrainEngineConfig(experiment_name="t", trial_name="t", path="", init_from_scratch=True,
                                              dtype="float32", model_preset="tiny-qwen2",
                                              optimizer=OptimizerConfig(lr=1e-3, warmup_steps_proportion=0.0)))
        e.create_process_group()
        e.initialize(None, FinetuneSpec(1, 48, 8), seed=seed)
        return e

    ft = FinetuneSpec(1, 48, 8)
    rc = RecoverConfig(experiment_name="t", trial_name="t", fileroot=str(tmp_path), mode="auto", freq_steps=1)
    a = make(3)
    a.train_batch(batch_of(0), loss_fn, lambda mb: float(mb["loss_mask"].sum()))
    a.set_version(1)
    import random

    import numpy as np

    assert RecoverHandler(rc, ft).dump(a, StepInfo(0, 0, 0, 6), force=True)
    # what the generators would have produced next, had the run gone on
    expect = (random.random(), float(np.random.rand()), torch.rand(3))
    ckpt = RecoverHandler(rc, ft)._ckpt_path()
    assert os.path.exists(os.path.join(ckpt, "rng", "rank00000.pt")), "every rank's generator states are in it"
    assert os.path.exists(os.path.join(ckpt, ".metadata")), "the recover checkpoint is a DCP directory"
    b = make(9)
    info = RecoverHandler(rc, ft).load(b)
    assert info is not None and b.get_version() == 1 and b.optimizer.step_count == 1
    got = (random.random(), float(np.random.rand()), torch.rand(3))       # the streams continue where they were
    assert got[0] == expect[0] and got[1] == expect[1] and torch.equal(got[2], expect[2])
    assert torch.equal(a.flat.flat, b.flat.flat) and torch.equal(a.optimizer.exp_avg, b.optimizer.exp_avg)
    sa = a.train_batch(batch_of(1), loss_fn, lambda mb: float(mb["loss_mask"].sum()))
    sb = b.train_batch(batch_of(1), loss_fn, lambda mb: float(mb["loss_mask"].sum()))
    assert sa["loss"] == sb["loss"] and torch.equal(a.flat.flat, b.flat.flat)


@pytest.mark.parametrize("n,flags", [(2, ["--tp", "2"]), (4, ["--tp", "2", "--pp", "2"])])
def test_lora_adapter_file_is_the_same_under_model_parallelism(tmp_path, n, flags):
    """Two training steps with adapters under tensor (and pipeline) parallelism write the PEFT adapter file and the
    merged model that one process writes: factors split over tensor-parallel ranks are gathered, the stages'
    adapters end up in one file."""
    from safetensors.torch import load_file

    from areal_b200.utils.hf_io import iter_hf_tensors

    one, par = str(tmp_path / "one"), str(tmp_path / "par")
    common = ["--phase", "train", "--format", "hf", "--lora", "--preset", "tiny-qwen2-4l", "--n-mbs", "2"]
    _run(1, 0, common + ["--dir", one])
    _run(n, 0, common + ["--dir", par] + flags)
    a = load_file(os.path.join(one, "ckpt", "adapter_model.safetensors"))
    b = load_file(os.path.join(par, "ckpt", "adapter_model.safetensors"))
    assert set(a) == set(b) and len(a) == 6 * 3 * 2          # 6 layers x (q, v, down) x (A, B)
    for k in a:
        assert a[k].shape == b[k].shape, k
        # A's first gradients are products with B = 0 plus rounding: Adam turns that noise into steps of up to
        # lr = 2e-3 per element in either direction, so A may differ by a few 1e-5 between layouts
        assert (a[k].double() - b[k].double()).abs().max() <= 1e-3 * a[k].abs().max() + 5e-5, k
    assert any(v.abs().max() > 0 for k, v in a.items() if "lora_B" in k)   # the adapters did train
    wa, wb = dict(iter_hf_tensors(os.path.join(one, "ckpt"))), dict(iter_hf_tensors(os.path.join(par, "ckpt")))
    assert set(wa) == set(wb)
    for k in wa:
        assert (wa[k].double() - wb[k].double()).abs().max() <= 1e-3 * wa[k].abs().max() + 5e-5, k
