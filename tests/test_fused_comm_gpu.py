"""Symmetric-memory collectives and fused GEMM+collective kernels vs NCCL (needs >= 2 GPUs),
and the bounded device-side wait (1 GPU: a flag that nothing sets)."""
import ctypes
import json
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.gpu
@pytest.mark.multi_gpu
def test_fused_comm_matches_nccl(tmp_path):
    n = min(torch.cuda.device_count(), 4)
    n = 2 if n < 4 else n
    out = str(tmp_path / "res.json")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", "29733",
           os.path.join(ROOT, "tests", "torchrun", "run_fused_comm.py"), out]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    res = json.load(open(out))
    assert res["ok"], res
    assert res["status"] == 0 and res["status_end"] == 0
    for k in ("all_gather_err", "all_to_all_err"):
        assert res[k] == 0.0, (k, res[k])
    assert res["reduce_scatter_err"] < 1e-4 and res["all_reduce_err"] < 1e-4
    assert res["a2a_gemm_repeat_err"] == 0.0
    for k in ("gemm_rs_err", "ag_gemm_err", "gemm_a2a_err", "gemm_rs_mixed_shapes_err", "a2a_gemm_err"):
        assert res[k] < 2e-2, (k, res[k])


@pytest.mark.gpu
def test_bounded_peer_wait_times_out_and_context_survives():
    """A barrier whose second participant never signals: the kernel gives up after its
    deadline, reports kErrPeerFlagTimeout through the status word, and the context stays usable."""
    from areal_b200.ops import _lib

    lib = _lib.kernels()
    lib.b200_ensure_device(ctypes.c_int(0))
    assert _lib.read_status() == 0
    flags = torch.zeros(64, dtype=torch.int32, device="cuda")
    other = torch.zeros(64, dtype=torch.int32, device="cuda")  # stands in for a peer that never answers
    table = (ctypes.c_void_p * 2)(flags.data_ptr(), other.data_ptr())
    rc = lib.b200_symm_barrier(table, ctypes.c_int(0), ctypes.c_int(2), ctypes.c_uint(1), _lib.stream_ptr())
    assert rc == 0
    assert _lib.read_status() == 4  # kErrPeerFlagTimeout
    assert _lib.read_status() == 0  # cleared
    x = torch.ones(1024, device="cuda")
    assert float((x * 2).sum()) == 2048.0


@pytest.mark.gpu
@pytest.mark.parametrize("rank", [0, 2])
def test_kchunk_gated_gemm_single_gpu(rank):
    """The all-to-all → GEMM kernel with four emulated source ranks on one GPU: the gather buffer holds
    the chunks [world, M, Kc], every flag already carries the epoch, and the K loop starts at chunk
    `rank`; the result must equal the plain product over the concatenated reduction dimension."""
    from areal_b200.ops import _lib

    lib = _lib.kernels()
    world, M, Kc, N = 4, 300, 128, 520
    torch.manual_seed(rank)
    chunks = (torch.randn(world, M, Kc, device="cuda") * 0.1).bfloat16()
    w = (torch.randn(N, world * Kc, device="cuda") * 0.1).bfloat16()
    flags = torch.full((64,), 7, dtype=torch.int32, device="cuda")
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    rc = lib.b200_gemm_kchunk_gated(_lib.ptr(chunks), _lib.ptr(w), _lib.ptr(out), _lib.ptr(flags), ctypes.c_uint(7),
                                    ctypes.c_int(world), ctypes.c_int(rank), ctypes.c_int(M), ctypes.c_int(N),
                                    ctypes.c_int(Kc), ctypes.c_longlong(w.stride(0)), ctypes.c_longlong(out.stride(0)),
                                    _lib.stream_ptr())
    assert rc == 0
    torch.cuda.synchronize()
    assert _lib.read_status() == 0
    ref = chunks.permute(1, 0, 2).reshape(M, world * Kc).float() @ w.float().t()
    assert float((out.float() - ref).abs().max() / ref.abs().max()) < 1e-2
