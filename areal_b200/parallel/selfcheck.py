"""Self-check of the symmetric-memory collectives and the fused compute+collective GEMMs on the ranks of a
running job: every op is compared with its NCCL / PyTorch statement, then timed (CUDA events, maximum over
ranks) against the unfused form (this library's GEMM plus the NCCL collective) and against its roofline, the
slower of the GEMM at the measured dense bf16 peak and the bytes that must cross NVLink at the measured
peer-copy bandwidth. The benchmark runs it outside its timed region whenever it has two or more ranks, and
the multi-GPU tests call the same function, so the numbers in a benchmark line and in the tests come from one
code path. Roles in the reference: the NCCL collectives around the linears of tensor / Ulysses parallelism
(areal/models/fsdp/ulysses.py:153-204, areal/engine/fsdp_utils/parallel.py:219-367)."""

from __future__ import annotations

import os

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops.gemm import gemm
from . import fused_linear as FL
from .symm_mem import SymmComm


def _timed(fn, n=10, warm=3):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(n):
        fn()
    e.record()
    torch.cuda.synchronize()
    t = torch.tensor([s.elapsed_time(e) / n], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def fused_comm_check(M: int | None = None, K: int | None = None, N: int | None = None, iters: int = 10,
                     peak_flops: float = 1664.7e12, link_bytes_per_s: float = 770e9) -> dict:
    """Collective over the default process group (NCCL, one rank per GPU). Returns errors, the device status
    word, fused / unfused timings and roofline fractions; identical on every rank."""
    timed = lambda fn: _timed(fn, n=iters)
    rank, world = dist.get_rank(), dist.get_world_size()
    res = {"world": world}
    torch.manual_seed(1234 + rank)
    # ---- plain collectives over peer memory
    comm = SymmComm(64 << 20, None)
    x = torch.randn(1 << 16, device="cuda")
    ag = comm.all_gather(x)
    ref = [torch.empty_like(x) for _ in range(world)]
    dist.all_gather(ref, x)
    res["all_gather_err"] = float((ag - torch.cat(ref)).abs().max())
    y = torch.randn(world * 4096, device="cuda")
    rs = comm.reduce_scatter(y)
    yr = y.clone(); dist.all_reduce(yr)
    res["reduce_scatter_err"] = float((rs - yr[rank * 4096:(rank + 1) * 4096]).abs().max())
    z = torch.randn(33, device="cuda")
    ar = comm.all_reduce_small(z)
    zr = z.clone(); dist.all_reduce(zr)
    res["all_reduce_err"] = float((ar - zr).abs().max())
    a = torch.randn(world * 1024, device="cuda")
    a2a = comm.all_to_all(a)
    ar2 = torch.empty_like(a)
    dist.all_to_all_single(ar2, a)
    res["all_to_all_err"] = float((a2a - ar2).abs().max())
    # ---- fused GEMM + collective
    K = int(K or os.environ.get("FUSED_K", 2048))
    N = int(N or os.environ.get("FUSED_N", 4096))
    M = int(M or os.environ.get("FUSED_M", 2048 * world))
    ctx = FL.FusedCommContext(None, max(M * max(K, N) * 2, 8 << 20) * 2)
    xs = (torch.randn(M, K // world, device="cuda") * 0.1).bfloat16()
    ws = (torch.randn(N, K // world, device="cuda") * 0.1).bfloat16()
    out = FL.gemm_reduce_scatter(ctx, xs, ws)
    ref = FL.gemm_reduce_scatter_ref(xs, ws, None)
    res["gemm_rs_err"] = float((out.float() - ref.float()).abs().max() / ref.float().abs().max())
    # calls of different shapes share the arrival counters: interleave them
    worst = 0.0
    for (m2, n2) in ((M // 2, N // 2), (M, N), (M // 2, N), (M, N // 2), (M // 2, N // 2)):
        xa = (torch.randn(m2, K // world, device="cuda") * 0.1).bfloat16()
        wa = (torch.randn(n2, K // world, device="cuda") * 0.1).bfloat16()
        o2 = FL.gemm_reduce_scatter(ctx, xa, wa)
        r2 = FL.gemm_reduce_scatter_ref(xa, wa, None)
        worst = max(worst, float((o2.float() - r2.float()).abs().max() / r2.float().abs().max()))
    res["gemm_rs_mixed_shapes_err"] = worst
    xl = (torch.randn(M // world, K, device="cuda") * 0.1).bfloat16()
    wc = (torch.randn(N // world, K, device="cuda") * 0.1).bfloat16()
    out = FL.all_gather_gemm(ctx, xl, wc)
    ref = FL.all_gather_gemm_ref(xl, wc, None)
    res["ag_gemm_err"] = float((out.float() - ref.float()).abs().max() / ref.float().abs().max())
    wq = (torch.randn(N, K, device="cuda") * 0.1).bfloat16()
    out = FL.gemm_all_to_all(ctx, xl, wq)
    ref = FL.gemm_all_to_all_ref(xl, wq, None)
    res["gemm_a2a_err"] = float((out.float() - ref.float()).abs().max() / ref.float().abs().max())
    # all-to-all → GEMM (Ulysses output projection): a [M, K/world] = all tokens x local heads
    ah = (torch.randn(M, K // world, device="cuda") * 0.1).bfloat16()
    wo = (torch.randn(N, K, device="cuda") * 0.1).bfloat16()
    out = FL.all_to_all_gemm(ctx, ah, wo)
    ref = FL.all_to_all_gemm_ref(ah, wo, None)
    res["a2a_gemm_err"] = float((out.float() - ref.float()).abs().max() / ref.float().abs().max())
    out2, chunks = FL.all_to_all_gemm(ctx, ah, wo, return_chunks=True)
    res["a2a_gemm_repeat_err"] = float((out2.float() - out.float()).abs().max())
    res["status"] = _lib.read_status()
    # ---- timings: fused vs NCCL + own GEMM
    res["t_gemm_rs_fused_ms"] = timed(lambda: FL.gemm_reduce_scatter(ctx, xs, ws))
    def unfused_rs():
        y = gemm(xs, ws)
        o = torch.empty((M // world, N), dtype=y.dtype, device="cuda")
        dist.reduce_scatter_tensor(o, y)
        return o
    res["t_gemm_rs_nccl_ms"] = timed(unfused_rs)
    res["t_ag_gemm_fused_ms"] = timed(lambda: FL.all_gather_gemm(ctx, xl, wc))
    def unfused_ag():
        full = torch.empty((M, K), dtype=xl.dtype, device="cuda")
        dist.all_gather_into_tensor(full, xl)
        return gemm(full, wc)
    res["t_ag_gemm_nccl_ms"] = timed(unfused_ag)
    res["t_gemm_a2a_fused_ms"] = timed(lambda: FL.gemm_all_to_all(ctx, xl, wq))
    def unfused_a2a():
        y = gemm(xl, wq)
        send = y.view(M // world, world, N // world).transpose(0, 1).contiguous()
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send)
        return recv
    res["t_gemm_a2a_nccl_ms"] = timed(unfused_a2a)
    res["t_a2a_gemm_fused_ms"] = timed(lambda: FL.all_to_all_gemm(ctx, ah, wo))
    def unfused_a2a_gemm():
        send = ah.view(world, M // world, K // world)
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send)
        return gemm(recv.permute(1, 0, 2).reshape(M // world, K), wo)
    res["t_a2a_gemm_nccl_ms"] = timed(unfused_a2a_gemm)
    res["shape"] = dict(M=M, K=K, N=N)
    # roofline per op: the slower of the GEMM at the measured cuBLAS peak and the bytes that must cross
    # NVLink at the measured peer-copy bandwidth (per direction per GPU)
    link = link_bytes_per_s
    frac = (world - 1) / world
    roof = {
        "gemm_rs": max(2.0 * M * N * (K // world) / peak_flops, frac * M * N * 2 / link),
        "ag_gemm": max(2.0 * M * (N // world) * K / peak_flops, frac * M * K * 2 / link),
        "gemm_a2a": max(2.0 * (M // world) * N * K / peak_flops, frac * (M // world) * N * 2 / link),
        "a2a_gemm": max(2.0 * (M // world) * N * K / peak_flops, frac * M * (K // world) * 2 / link),
    }
    for k, t in roof.items():
        res[f"roofline_{k}_ms"] = t * 1e3
        res[f"frac_of_roofline_{k}_fused"] = t * 1e3 / res[f"t_{k}_fused_ms"]
        res[f"frac_of_roofline_{k}_nccl"] = t * 1e3 / res[f"t_{k}_nccl_ms"]
    res["status_end"] = _lib.read_status()
    res["max_err"] = max(v for k, v in res.items() if k.endswith("_err"))
    # exact for pure data movement, fp32 rounding for reductions, bf16 rounding for the fused GEMMs
    res["ok"] = bool(
        res["status"] == 0 and res["status_end"] == 0 and res["all_gather_err"] == 0.0 and res["all_to_all_err"] == 0.0
        and res["reduce_scatter_err"] < 1e-4 and res["all_reduce_err"] < 1e-4 and res["a2a_gemm_repeat_err"] == 0.0
        and all(res[k] < 2e-2 for k in ("gemm_rs_err", "ag_gemm_err", "gemm_a2a_err", "gemm_rs_mixed_shapes_err",
                                         "a2a_gemm_err")))
    return res
