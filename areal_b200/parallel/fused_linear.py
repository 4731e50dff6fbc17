"""Fused compute + collective linears over NVLink peer memory
(``csrc/gemm_fused_comm.cu``) and their NCCL / gloo reference forms.

* :func:`gemm_reduce_scatter` – row-parallel linear (``K`` sharded): each rank's
  partial product is stored tile by tile into the owners' staging buffers from
  the GEMM epilogue, then summed locally. Tensor-parallel ``o_proj`` /
  ``down_proj`` with sequence-parallel outputs.
* :func:`all_gather_gemm` – column-parallel linear on sequence-sharded input:
  rows are pushed to the peers while the GEMM already works on the local rows;
  its TMA producer waits per source rank on an arrival flag. Tensor-parallel
  ``qkv`` / ``gate_up`` and the FSDP-style "gather then first GEMM".
* :func:`gemm_all_to_all` – Ulysses: the QKV projection's epilogue writes every
  head slice directly to the rank that owns those heads (sequence gathered).

A :class:`FusedCommContext` owns the symmetric staging / gather buffers, flags
and epochs for one process group. On CPU (gloo) the same functions run their
unfused reference, which is also the oracle of the GPU tests. Reference call
sites: areal/engine/fsdp_utils/parallel.py:219-367 (DTensor TP plan),
areal/models/fsdp/ulysses.py:153-204 (all-to-all).
"""

from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops.gemm import gemm
from .symm_mem import SymmBarrier, SymmBuffer


class FusedCommContext:
    def __init__(self, group: dist.ProcessGroup | None, max_stage_bytes: int, device=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.cuda = torch.cuda.is_available() and (device is None or torch.device(device).type == "cuda")
        self.max_stage_bytes = max_stage_bytes
        if self.cuda:
            self.stage = SymmBuffer(max_stage_bytes, group, device)
            self.gather = SymmBuffer(max_stage_bytes, group, device)
            self.flags = SymmBuffer(256, group, device)
            self.barrier = SymmBarrier(group, device)
            self.device = self.stage.device
            self._stage_tbl = self.stage.ptr_table()
            self._gather_tbl = self.gather.ptr_table()
            self._flag_tbl = self.flags.ptr_table()
            self._done = torch.zeros(1, dtype=torch.int32, device=self.device)
            # barrier-free reduce-scatter: two staging halves, one row-block counter array per half
            self.rs_counters = SymmBuffer(2 * 4096 * 4, group, device)
            self.rs_counters.tensor(torch.int32).zero_()
            self._rs_cnt_tbl = [self.rs_counters.ptr_table(byte_offset=h * 4096 * 4) for h in range(2)]
            self._rs_stage_tbl = [self.stage.ptr_table(byte_offset=h * (max_stage_bytes // 2)) for h in range(2)]
            self._rs_expected = torch.zeros((2, 4096 * 4), dtype=torch.int32, device=self.device)
            self._rs_calls = 0
            torch.cuda.synchronize(self.device)
            if self.world > 1:
                self.barrier.sync()  # the zeroed counters are visible before anybody adds to them
            self._epoch = 0
            self.side_stream = torch.cuda.Stream(self.device)

    def next_epoch(self) -> int:
        self._epoch += 1
        return self._epoch


# --------------------------------------------------------------------------- references


def gemm_reduce_scatter_ref(x, w, group):
    """``reduce_scatter_rows(x @ w.T)``; ``x [M, K/P]``, ``w [N, K/P]`` → ``[M/P, N]``."""
    y = (x.float() @ w.float().t())
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return y.to(x.dtype)
    out = torch.empty((y.shape[0] // world, y.shape[1]), dtype=y.dtype, device=y.device)
    dist.reduce_scatter_tensor(out, y.contiguous(), group=group) if y.is_cuda else _rs_cpu(out, y, group)
    return out.to(x.dtype)


def _rs_cpu(out, y, group):
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    dist.all_reduce(y, group=group)
    n = y.shape[0] // world
    out.copy_(y[rank * n:(rank + 1) * n])


def all_gather_gemm_ref(x, w, group):
    """``all_gather_rows(x) @ w.T``; ``x [M/P, K]``, ``w [N/P, K]`` → ``[M, N/P]``."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world > 1:
        parts = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(parts, x.contiguous(), group=group)
        x = torch.cat(parts, 0)
    return (x.float() @ w.float().t()).to(x.dtype)


def gemm_all_to_all_ref(x, w, group):
    """Ulysses projection: ``x [M, K]`` (local sequence shard), ``w [N, K]`` (all heads) →
    ``[P*M, N/P]`` (full sequence, this rank's head slice)."""
    y = (x.float() @ w.float().t()).to(x.dtype)
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return y
    M, N = y.shape
    send = [c.contiguous() for c in y.view(M, world, N // world).unbind(1)]
    recv = [torch.empty_like(send[0]) for _ in range(world)]
    if y.is_cuda:
        dist.all_to_all(recv, send, group=group)
    else:  # gloo has no all_to_all: gather every column block on its owner
        for r in range(world):
            dst = recv if dist.get_rank(group) == r else None
            dist.gather(send[r], dst, dst=dist.get_global_rank(group, r) if group is not None else r, group=group)
    return torch.cat(recv, 0)


def all_to_all_gemm_ref(a, w, group):
    """Ulysses output projection: ``a [P*M, Kc]`` (all tokens, this rank's heads), ``w [N, P*Kc]`` →
    ``[M, N]`` for this rank's tokens: the head→sequence exchange followed by the projection."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return (a.float() @ w.float().t()).to(a.dtype)
    M = a.shape[0] // world
    send = a.contiguous().view(world, M, a.shape[1])
    recv = torch.empty_like(send)
    if a.is_cuda:
        dist.all_to_all_single(recv, send, group=group)
    else:
        rank = dist.get_rank(group)
        for r in range(world):
            dst = list(recv.unbind(0)) if rank == r else None
            dist.gather(send[r].contiguous(), dst, dst=dist.get_global_rank(group, r) if group is not None else r,
                        group=group)
    full = recv.permute(1, 0, 2).reshape(M, -1)  # columns in source-rank order = head order
    return (full.float() @ w.float().t()).to(a.dtype)


# --------------------------------------------------------------------------- fused (CUDA)


def gemm_reduce_scatter(ctx: FusedCommContext, x: torch.Tensor, w: torch.Tensor, add: torch.Tensor | None = None):
    if not (ctx.cuda and x.is_cuda):
        y = gemm_reduce_scatter_ref(x, w, ctx.group)
        return y + add if add is not None else y
    M, K = x.shape
    N = w.shape[0]
    P = ctx.world
    assert M % P == 0 and M * N * 2 <= ctx.max_stage_bytes
    x = x if x.is_contiguous() else x.contiguous()
    lib = _lib.kernels()
    n_cnt = (M // P // 128) * (-(-N // 256)) if M % (P * 128) == 0 else 1 << 30
    if P > 1 and M % (P * 128) == 0 and N % 8 == 0 and 2 * M * N * 2 <= ctx.max_stage_bytes and n_cnt <= 4096:
        # single kernel, no barrier: peer tiles first (stored into the owners' staging half with arrival
        # counters), own tiles last (their epilogue adds the staged partials); halves alternate per call
        h = ctx._rs_calls & 1
        ctx._rs_calls += 1
        half = ctx.max_stage_bytes // 2
        out = torch.empty((M // P, N), dtype=x.dtype, device=x.device)
        rc = lib.b200_gemm_rs_fused(_lib.ptr(x), _lib.ptr(w), ctx._rs_stage_tbl[h], ctx._rs_cnt_tbl[h],
                                    ctypes.c_void_p(ctx.stage.local_ptr + h * half),
                                    ctypes.c_void_p(ctx.rs_counters.local_ptr + h * 4096 * 4),
                                    _lib.ptr(ctx._rs_expected[h]), _lib.ptr(add), _lib.ptr(out), ctypes.c_int(P),
                                    ctypes.c_int(ctx.rank), ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(K),
                                    ctypes.c_longlong(x.stride(0)), ctypes.c_longlong(w.stride(0)), _lib.stream_ptr())
        _lib.check(rc, "b200_gemm_rs_fused")
        _lib.count_launch()
        return out
    ctx.barrier.sync()  # peers are done reading their staging buffers from the previous call
    rc = lib.b200_gemm_peer_scatter(_lib.ptr(x), _lib.ptr(w), ctx._stage_tbl, ctypes.c_int(P), ctypes.c_int(ctx.rank),
                                    ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(K),
                                    ctypes.c_longlong(x.stride(0)), ctypes.c_longlong(w.stride(0)),
                                    ctypes.c_int(0), _lib.stream_ptr())
    _lib.check(rc, "b200_gemm_peer_scatter")
    ctx.barrier.sync()  # every rank's partial tiles have landed
    n = (M // P) * N
    out = torch.empty((M // P, N), dtype=x.dtype, device=x.device)
    rc = lib.b200_reduce_slices(ctypes.c_void_p(ctx.stage.local_ptr), _lib.ptr(add), _lib.ptr(out),
                                ctypes.c_int(P), ctypes.c_longlong(n), _lib.stream_ptr())
    _lib.check(rc, "b200_reduce_slices")
    _lib.count_launch(2)
    return out


def all_gather_gemm(ctx: FusedCommContext, x: torch.Tensor, w: torch.Tensor, return_gathered: bool = False):
    """With ``return_gathered`` also returns the gathered rows ``[M, K]``; on the fused path this is
    a view of the (local) gather buffer, valid until the next fused call on ``ctx``."""
    if return_gathered:
        if not (ctx.cuda and x.is_cuda) or x.shape[0] % 128 or ctx.world == 1:
            full = ctx_all_gather(ctx, x) if ctx.world > 1 else x
            y = gemm(full, w) if (full.is_cuda and full.dtype == torch.bfloat16) else (full.float() @ w.float().t()).to(x.dtype)
            return y, full
        y = all_gather_gemm(ctx, x, w)
        M = x.shape[0] * ctx.world
        return y, ctx.gather.tensor(x.dtype, M * x.shape[1]).view(M, x.shape[1])
    if not (ctx.cuda and x.is_cuda):
        return all_gather_gemm_ref(x, w, ctx.group)
    Ml, K = x.shape
    N = w.shape[0]
    P = ctx.world
    M = Ml * P
    if Ml % 128 or P == 1:
        # tile rows must not straddle source ranks; small / odd shapes take the unfused path
        full = ctx_all_gather(ctx, x) if P > 1 else x
        return gemm(full, w)
    assert M * K * 2 <= ctx.max_stage_bytes
    x = x if x.is_contiguous() else x.contiguous()
    lib = _lib.kernels()
    epoch = ctx.next_epoch()
    gather = ctx.gather.tensor(x.dtype, M * K).view(M, K)
    ctx.barrier.sync()  # nobody still reads the gather buffer of the previous call
    cur = torch.cuda.current_stream()
    gather[ctx.rank * Ml:(ctx.rank + 1) * Ml].copy_(x)
    ctx.side_stream.wait_stream(cur)
    with torch.cuda.stream(ctx.side_stream):
        rc = lib.b200_push_chunks(ctx._gather_tbl, ctx._flag_tbl, ctypes.c_int(P), ctypes.c_int(ctx.rank),
                                  _lib.ptr(x), ctypes.c_longlong(Ml * K * 2),
                                  ctypes.c_longlong(ctx.rank * Ml * K * 2), ctypes.c_uint(epoch),
                                  _lib.ptr(ctx._done), _lib.stream_ptr())
        _lib.check(rc, "b200_push_chunks")
    out = torch.empty((M, N), dtype=x.dtype, device=x.device)
    rc = lib.b200_gemm_gated(ctypes.c_void_p(ctx.gather.local_ptr), _lib.ptr(w), _lib.ptr(out),
                             ctypes.c_void_p(ctx.flags.local_ptr), ctypes.c_uint(epoch), ctypes.c_int(P),
                             ctypes.c_int(ctx.rank), ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(K),
                             ctypes.c_longlong(K), ctypes.c_longlong(w.stride(0)), ctypes.c_longlong(N),
                             _lib.stream_ptr())
    _lib.check(rc, "b200_gemm_gated")
    cur.wait_stream(ctx.side_stream)
    x.record_stream(ctx.side_stream)
    _lib.count_launch(2)
    return out


def ctx_all_gather(ctx: FusedCommContext, x: torch.Tensor) -> torch.Tensor:
    out = torch.empty((ctx.world * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(out, x.contiguous(), group=ctx.group) if x.is_cuda else \
        dist.all_gather(list(out.chunk(ctx.world, 0)), x.contiguous(), group=ctx.group)
    return out


def gemm_all_to_all(ctx: FusedCommContext, x: torch.Tensor, w: torch.Tensor):
    if not (ctx.cuda and x.is_cuda) or ctx.world == 1:
        return gemm_all_to_all_ref(x, w, ctx.group)
    M, K = x.shape
    N = w.shape[0]
    P = ctx.world
    assert N % P == 0 and P * M * (N // P) * 2 <= ctx.max_stage_bytes
    x = x if x.is_contiguous() else x.contiguous()
    lib = _lib.kernels()
    ctx.barrier.sync()
    rc = lib.b200_gemm_peer_scatter(_lib.ptr(x), _lib.ptr(w), ctx._stage_tbl, ctypes.c_int(P), ctypes.c_int(ctx.rank),
                                    ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(K),
                                    ctypes.c_longlong(x.stride(0)), ctypes.c_longlong(w.stride(0)),
                                    ctypes.c_int(1), _lib.stream_ptr())
    _lib.check(rc, "b200_gemm_peer_scatter")
    ctx.barrier.sync()
    _lib.count_launch()
    return ctx.stage.tensor(x.dtype, P * M * (N // P)).view(P * M, N // P).clone()


def all_to_all_gemm(ctx: FusedCommContext, a: torch.Tensor, w: torch.Tensor, return_chunks: bool = False):
    """``head_to_seq(a) @ w.T`` in one GEMM kernel whose reduction dimension is split by source rank:
    every rank pushes the row block of each destination into that rank's gather buffer (peer stores,
    one arrival flag per source), and the GEMM's TMA producer starts with the local chunk and waits for
    a peer's chunk only when its K loop reaches it, so the exchange overlaps the math. With
    ``return_chunks`` also returns the received operand ``[P, M, Kc]`` (a copy; for the backward)."""
    P = ctx.world
    Kc = a.shape[1]
    M = a.shape[0] // P
    if not (ctx.cuda and a.is_cuda) or P == 1 or Kc % 64 or a.dtype != torch.bfloat16 or \
            a.numel() * 2 > ctx.max_stage_bytes:
        y = all_to_all_gemm_ref(a, w, ctx.group)
        return (y, None) if return_chunks else y
    N = w.shape[0]
    a = a if a.is_contiguous() else a.contiguous()
    w = w if w.is_contiguous() else w.contiguous()
    lib = _lib.kernels()
    epoch = ctx.next_epoch()
    gather = ctx.gather.tensor(a.dtype, P * M * Kc).view(P, M, Kc)
    ctx.barrier.sync()  # nobody still reads the gather buffer of the previous call
    cur = torch.cuda.current_stream()
    gather[ctx.rank].copy_(a[ctx.rank * M:(ctx.rank + 1) * M])
    if not hasattr(ctx, "_a2a_done"):
        ctx._a2a_done = torch.zeros(8, dtype=torch.int32, device=ctx.device)
    ctx.side_stream.wait_stream(cur)
    with torch.cuda.stream(ctx.side_stream):
        rc = lib.b200_push_a2a(ctx._gather_tbl, ctx._flag_tbl, ctypes.c_int(P), ctypes.c_int(ctx.rank), _lib.ptr(a),
                               ctypes.c_longlong(M * Kc * 2), ctypes.c_uint(epoch), _lib.ptr(ctx._a2a_done),
                               _lib.stream_ptr())
        _lib.check(rc, "b200_push_a2a")
    out = torch.empty((M, N), dtype=a.dtype, device=a.device)
    rc = lib.b200_gemm_kchunk_gated(ctypes.c_void_p(ctx.gather.local_ptr), _lib.ptr(w), _lib.ptr(out),
                                    ctypes.c_void_p(ctx.flags.local_ptr), ctypes.c_uint(epoch), ctypes.c_int(P),
                                    ctypes.c_int(ctx.rank), ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(Kc),
                                    ctypes.c_longlong(w.stride(0)), ctypes.c_longlong(out.stride(0)),
                                    _lib.stream_ptr())
    _lib.check(rc, "b200_gemm_kchunk_gated")
    cur.wait_stream(ctx.side_stream)
    _lib.count_launch(2)
    if return_chunks:
        return out, gather.clone()
    return out
