"""Functional oracle for the whole rollout → train → weight-update step: the tiny
Qwen2-architecture GRPO configuration on CPU with gloo, two ranks, fp32, seed 0."""
import json
import os
import subprocess
import sys

import pytest

from tests.conftest import free_port

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(tmp_path, mode, nproc, port, preset="tiny-qwen2"):
    out = str(tmp_path / f"res_{mode}")
    env = dict(os.environ, AREAL_B200_FILEROOT=str(tmp_path), OMP_NUM_THREADS="2", AREAL_LOG_LEVEL="WARNING",
               AREAL_B200_TEST_PRESET=preset)
    env.pop("CUDA_VISIBLE_DEVICES", None)
    env["CUDA_VISIBLE_DEVICES"] = ""
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(free_port()),
           os.path.join(ROOT, "tests", "torchrun", "run_grpo_cfg1.py"), out, mode]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    return [json.load(open(f"{out}.{i}")) for i in range(nproc)]


@pytest.mark.slow
def test_colocated_two_ranks(tmp_path):
    res = _run(tmp_path, "colocated", 2, 29611)
    a, b = res
    assert a["steps"] == b["steps"] == 2 and a["version"] == b["version"] == 2
    # data-parallel ranks hold identical weights after the sharded optimizer steps
    assert a["checksum"] == pytest.approx(b["checksum"], rel=1e-9, abs=1e-9)
    assert a["absum"] == pytest.approx(b["absum"], rel=1e-9)
    assert a["grad_norm"] == pytest.approx(b["grad_norm"], rel=1e-5)
    assert all(g > 0 for g in a["grad_norm"])
    # the rollout engine of every rank received the new weights and version
    assert a["rollout_matches"] and b["rollout_matches"]
    assert a["rollout_version"] == b["rollout_version"] == 2
    assert sum(a["tokens"]) > 0
    assert all(r is not None and 0.0 <= r <= 1.0 for r in a["eval_reward"])


@pytest.mark.slow
@pytest.mark.parametrize("mode,preset", [("colocated", "tiny-deepseek-v3"), ("disagg", "tiny-deepseek-v3"),
                                         ("colocated", "tiny-bailing-hybrid")])
def test_latent_and_lightning_attention_families_train_and_generate_in_one_job(tmp_path, mode, preset):
    """Latent attention + grouped sigmoid routing (and lightning layers with their per-sequence state) through the
    whole loop: the rollout engine generates, the trainer steps, the new weights reach the engine (a flat copy when
    colocated, pushed to the rollout rank otherwise)."""
    res = _run(tmp_path, mode, 2, 0, preset=preset)
    trainers = [r for r in res if r["is_trainer"]]
    assert all(r["steps"] == 2 and r["version"] == 2 and all(g > 0 for g in r["grad_norm"]) for r in trainers)
    assert all(r["rollout_version"] == 2 for r in res if "rollout_version" in r)
    if mode == "colocated":
        assert all(r["rollout_matches"] for r in trainers)
        assert trainers[0]["checksum"] == pytest.approx(trainers[1]["checksum"], rel=1e-9, abs=1e-9)
    assert sum(trainers[0]["tokens"]) > 0


@pytest.mark.slow
def test_disaggregated_two_ranks(tmp_path):
    res = _run(tmp_path, "disagg", 2, 29612)
    gen = next(r for r in res if not r["is_trainer"])
    tr = next(r for r in res if r["is_trainer"])
    assert tr["steps"] == 2 and tr["version"] == 2
    assert gen["rollout_version"] == 2
    assert all(g > 0 for g in tr["grad_norm"])
    # evaluation runs on the rollout rank (it holds the validation set) and reports to the trainer after every step
    assert len(tr["eval_reward"]) == 2 and all(r is not None and 0.0 <= r <= 1.0 for r in tr["eval_reward"])


@pytest.mark.slow
def test_disaggregated_four_ranks(tmp_path):
    """Two rollout ranks feed two data-parallel trainer ranks: both trainers end with the same weights, both rollout
    engines reach the trainer's version, and the evaluation result is the same on every trainer (summed over the
    rollout ranks that ran it)."""
    res = _run(tmp_path, "disagg", 4, 29613)
    gens = [r for r in res if not r["is_trainer"]]
    trs = [r for r in res if r["is_trainer"]]
    assert len(gens) == 2 and len(trs) == 2
    assert all(g["rollout_version"] == 2 for g in gens)
    a, b = trs
    assert a["steps"] == b["steps"] == 2 and a["version"] == b["version"] == 2
    assert a["checksum"] == pytest.approx(b["checksum"], rel=1e-9, abs=1e-9)
    assert a["grad_norm"] == pytest.approx(b["grad_norm"], rel=1e-5)
    assert a["eval_reward"] == b["eval_reward"] and all(r is not None for r in a["eval_reward"])
