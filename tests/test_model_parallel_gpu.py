"""Tensor / Ulysses / pipeline / expert parallelism on real GPUs (NCCL + the fused peer-memory
kernels): one optimizer step on 2 ranks must reproduce the single-GPU loss, gradient norm and
gradients within bf16 tolerance."""
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
WORKER = os.path.join(ROOT, "tests", "torchrun", "run_model_parallel.py")

pytestmark = [pytest.mark.gpu, pytest.mark.multi_gpu]


def _run(cmd):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2500:] + r.stderr[-3500:]
    return r.stdout


@pytest.mark.parametrize("args,preset,n_mbs", [(["--tp", "2"], "tiny-qwen2", 1), (["--sp", "2"], "tiny-qwen2", 1),
                                               (["--sp", "2", "--no-bias"], "tiny-qwen2", 1),
                                               (["--sp", "2", "--zigzag"], "tiny-qwen2", 1),
                                               (["--pp", "2"], "tiny-qwen2", 2), (["--ep", "2"], "tiny-qwen3-moe", 1),
                                               (["--pp", "2", "--vpp", "2"], "tiny-qwen2-4l", 4),
                                               (["--pp", "2", "--schedule", "ZB1P"], "tiny-qwen2-4l", 4),
                                               (["--tp", "2", "--ep", "2"], "tiny-qwen3-moe", 1),
                                               (["--tp", "2", "--etp", "2"], "tiny-qwen3-moe", 1),
                                               (["--tp", "2", "--lora"], "tiny-qwen2-4l", 1)])
def test_two_gpu_step_matches_one_gpu(tmp_path, args, preset, n_mbs):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    ref = str(tmp_path / "ref.pt")
    shared = [a for a in args if a in ("--no-bias", "--lora")]   # flags that the single-GPU reference run takes too
    common = ["--device", "cuda", "--preset", preset, "--n-mbs", str(n_mbs)] + shared
    args = [a for a in args if a not in shared]
    env_free = [sys.executable, WORKER, "--ref"] + common + [ref]
    clean = {k: v for k, v in os.environ.items() if k not in ("RANK", "WORLD_SIZE", "LOCAL_RANK")}
    r = subprocess.run(env_free, env=clean, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    out = _run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
                "127.0.0.1", "--master-port", "29781", WORKER] + args + common + [ref])
    assert "OK" in out
