"""Fused LM-head → per-token logprob / entropy, vocab-parallel ready.

``lm_head_logprobs(x, w, labels, temperature)`` returns ``(logp [T], entropy [T])``
of ``softmax(x w^T / temperature)`` at ``labels`` without ever materialising the
``[T, V]`` logits on the CUDA path (``csrc/lm_head.cu``). Under tensor
parallelism every rank holds a contiguous vocabulary shard of ``w``; the
per-split partial statistics are exchanged (a few floats per token) and merged
by the same combine kernel, replacing the reference's 3-4 all-reduces over
``[T]`` (areal/utils/functional/vocab_parallel.py:84-372).

Backward recomputes the logits of one row chunk at a time, writes ``d logits``
for that chunk only (bf16 scratch) and feeds two plain GEMMs (dX, dW).
"""

from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from . import _lib
from .gemm import gemm

_BWD_ROW_CHUNK = 4096


def lm_head_logprobs_ref(x, w, labels, temperature=1.0, tp_group=None, vocab_start=0):
    """fp32 reference (also the CPU path). With ``tp_group`` the local shard's
    statistics are all-reduced like the reference implementation does."""
    logits = (x.float() @ w.float().t()) / temperature
    if tp_group is None or dist.get_world_size(tp_group) == 1:
        lse = torch.logsumexp(logits, -1)
        tgt = logits.gather(-1, labels.long()[:, None]).squeeze(-1)
        p = torch.softmax(logits, -1)
        ent = lse - (p * logits).sum(-1)
        return tgt - lse, ent
    # vocab-parallel: max → sum-exp → target → sum p*x
    V = logits.shape[1]
    mx = logits.max(-1).values.detach()
    dist.all_reduce(mx, op=dist.ReduceOp.MAX, group=tp_group)
    ex = (logits - mx[:, None]).exp()
    se = _AllReduceSum.apply(ex.sum(-1), tp_group)
    local = labels.long() - vocab_start
    ok = (local >= 0) & (local < V)
    tgt = logits.gather(-1, local.clamp(0, V - 1)[:, None]).squeeze(-1) * ok
    tgt = _AllReduceSum.apply(tgt, tp_group)
    lse = mx + se.log()
    sx = _AllReduceSum.apply((ex * logits).sum(-1), tp_group) / se
    return tgt - lse, lse - sx


class _AllReduceSum(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        x = x.clone()
        dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


class _LMHead(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, labels, temperature, tp_group, vocab_start, tp_fused=None):
        T, H = x.shape
        V = w.shape[0]
        x = x if x.is_contiguous() else x.contiguous()
        labels = labels.to(torch.int32).contiguous()
        lib = _lib.kernels()
        lib.b200_lm_head_nsplit.restype = ctypes.c_int
        nsplit = lib.b200_lm_head_nsplit(ctypes.c_int(T), ctypes.c_int(V))
        inv_t = 1.0 / float(temperature)
        tp = dist.get_world_size(tp_group) if tp_group is not None else 1
        if tp > 1 and tp_fused is not None and getattr(tp_fused, "cuda", False):
            # vocab-parallel, fused: the GEMM epilogue stores every row's (max, sum-exp, sum x·exp, target)
            # record into all tp peers' buffers over NVLink, so the exchange of the softmax statistics is
            # part of the kernel; one device-side barrier later every rank combines its local copy.
            # Buffers alternate between calls: a rank can only be one barrier ahead of the slowest, so
            # the copy being combined is never overwritten.
            bufs, tables, calls = _peer_partials(tp_fused, tp * nsplit * T * 16)
            h = calls & 1
            rc = lib.b200_lm_head_stats_peers(_lib.ptr(x), _lib.ptr(w), _lib.ptr(labels), tables[h], ctypes.c_int(tp),
                                              ctypes.c_int(tp_fused.rank), ctypes.c_int(T), ctypes.c_int(V),
                                              ctypes.c_int(H), ctypes.c_longlong(x.stride(0)),
                                              ctypes.c_longlong(w.stride(0)), ctypes.c_int(vocab_start),
                                              ctypes.c_float(inv_t), _lib.stream_ptr())
            _lib.check(rc, "b200_lm_head_stats_peers")
            tp_fused.barrier.sync()
            half = bufs.nbytes // 2
            partials = bufs.tensor(torch.float32, tp * nsplit * T * 4, byte_offset=h * half).view(tp * nsplit, T, 4)
            return _LMHead._finish(ctx, lib, partials, tp * nsplit, x, w, labels, inv_t, tp_group, vocab_start)
        partials = torch.empty((nsplit, T, 4), dtype=torch.float32, device=x.device)
        lib.b200_lm_head_stats.restype = ctypes.c_int
        rc = lib.b200_lm_head_stats(_lib.ptr(x), _lib.ptr(w), _lib.ptr(labels), _lib.ptr(partials),
                                    ctypes.c_int(T), ctypes.c_int(V), ctypes.c_int(H),
                                    ctypes.c_longlong(x.stride(0)), ctypes.c_longlong(w.stride(0)),
                                    ctypes.c_int(vocab_start), ctypes.c_float(inv_t),
                                    _lib.stream_ptr())
        _lib.check(rc, "b200_lm_head_stats")
        if tp > 1:
            # ranks may pick different split counts only if their shard sizes differ; pad to max
            ns = torch.tensor([nsplit], device=x.device)
            dist.all_reduce(ns, op=dist.ReduceOp.MAX, group=tp_group)
            nmax = int(ns.item())
            if nmax != nsplit:
                pad = torch.zeros((nmax - nsplit, T, 4), dtype=torch.float32, device=x.device)
                pad[..., 0] = float("-inf")
                partials = torch.cat([partials, pad], 0)
            gathered = torch.empty((tp * nmax, T, 4), dtype=torch.float32, device=x.device)
            dist.all_gather_into_tensor(gathered, partials.contiguous(), group=tp_group)
            partials, nparts = gathered, tp * nmax
        else:
            nparts = nsplit
        return _LMHead._finish(ctx, lib, partials, nparts, x, w, labels, inv_t, tp_group, vocab_start)

    @staticmethod
    def _finish(ctx, lib, partials, nparts, x, w, labels, inv_t, tp_group, vocab_start):
        T = x.shape[0]
        logp = torch.empty(T, dtype=torch.float32, device=x.device)
        ent = torch.empty_like(logp)
        logz = torch.empty_like(logp)
        ey = torch.empty_like(logp)
        lib.b200_lm_head_combine.restype = ctypes.c_int
        rc = lib.b200_lm_head_combine(_lib.ptr(partials), ctypes.c_int(nparts), ctypes.c_int(T),
                                      _lib.ptr(logp), _lib.ptr(ent), _lib.ptr(logz), _lib.ptr(ey),
                                      _lib.stream_ptr())
        _lib.check(rc, "b200_lm_head_combine")
        _lib.count_launch(2)
        ctx.save_for_backward(x, w, labels, logz, ey)
        ctx.inv_t = inv_t
        ctx.tp_group = tp_group
        ctx.vocab_start = vocab_start
        return logp, ent

    @staticmethod
    def backward(ctx, g_logp, g_ent):
        x, w, labels, logz, ey = ctx.saved_tensors
        T, H = x.shape
        V = w.shape[0]
        lib = _lib.kernels()
        lib.b200_lm_head_dlogits.restype = ctypes.c_int
        g_logp = g_logp.float().contiguous() if g_logp is not None else None
        g_ent = g_ent.float().contiguous() if g_ent is not None else None
        need_dx, need_dw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        dx = torch.empty_like(x) if need_dx else None
        main = getattr(w, "main_grad", None)
        dw_acc = main if main is not None else (
            torch.zeros((V, H), dtype=torch.float32, device=x.device) if need_dw else None)
        Vp = (V + 7) // 8 * 8
        chunk = min(T, _BWD_ROW_CHUNK)
        dz = torch.empty((chunk, Vp), dtype=torch.bfloat16, device=x.device)
        for r0 in range(0, T, chunk):
            r1 = min(T, r0 + chunk)
            n = r1 - r0
            xs = x[r0:r1]
            rc = lib.b200_lm_head_dlogits(
                _lib.ptr(xs), _lib.ptr(w), _lib.ptr(labels[r0:r1]),
                _lib.ptr(g_logp[r0:r1]) if g_logp is not None else None,
                _lib.ptr(g_ent[r0:r1]) if g_ent is not None else None,
                _lib.ptr(logz[r0:r1]), _lib.ptr(ey[r0:r1]), _lib.ptr(dz),
                ctypes.c_int(n), ctypes.c_int(V), ctypes.c_int(H),
                ctypes.c_longlong(x.stride(0)), ctypes.c_longlong(w.stride(0)),
                ctypes.c_longlong(Vp), ctypes.c_int(ctx.vocab_start), ctypes.c_float(ctx.inv_t),
                _lib.stream_ptr())
            _lib.check(rc, "b200_lm_head_dlogits")
            _lib.count_launch()
            dzv = dz[:n, :V]
            if need_dx:
                gemm(dzv, w, b_mn=True, out=dx[r0:r1])
            if need_dw:
                gemm(dzv, xs, a_mn=True, b_mn=True, out=dw_acc, accumulate=True)
        # With a vocabulary shard, dx is this rank's PARTIAL input gradient (like the reference
        # restatement above): the caller's gather of the token shards sums the partials in its
        # backward (reduce-scatter), which moves half the bytes of an all-reduce here.
        dw = None
        if need_dw and main is None:
            dw = dw_acc.to(w.dtype)
        return dx, dw, None, None, None, None, None


def _peer_partials(fctx, nbytes: int):
    """Two symmetric buffers (one allocation, halves alternate per call) for the vocab-parallel
    statistics, sized on first use and grown collectively when a larger micro-batch arrives (every
    rank of the group sees the same shapes, so every rank reallocates at the same call)."""
    from ..parallel.symm_mem import SymmBuffer

    st = getattr(fctx, "_lm_partials", None)
    need = (nbytes + 255) // 256 * 256
    if st is None or st[0].nbytes < 2 * need:
        if st is not None:
            fctx.barrier.sync()
            torch.cuda.synchronize(fctx.device)
            st[0].close()
        size = 2 * max(need, 1 << 20)
        buf = SymmBuffer(size, fctx.group, fctx.device)
        st = [buf, [buf.ptr_table(byte_offset=h * (size // 2)) for h in range(2)], 0]
        fctx._lm_partials = st
    calls = st[2]
    st[2] += 1
    return st[0], st[1], calls


def lm_head_logprobs(x, w, labels, temperature: float = 1.0, tp_group=None, vocab_start: int = 0, tp_fused=None):
    """Per-token log-probability of ``labels`` and entropy of the next-token
    distribution ``softmax(x @ w.T / temperature)``. ``w`` may be this rank's
    vocabulary shard starting at global id ``vocab_start``; the gradient with respect to ``x``
    is then this shard's partial contribution, to be summed over ``tp_group`` by the caller
    (``parallel.tensor_parallel.gather_seq`` does so in its backward). With ``tp_fused`` (the tp group's
    ``FusedCommContext``) the statistics are exchanged by peer stores from the GEMM epilogue instead
    of an NCCL all-gather."""
    if _lib.use_cuda_kernels(x, w) and x.dtype == torch.bfloat16 and x.shape[1] % 8 == 0:
        return _LMHead.apply(x, w, labels, temperature, tp_group, vocab_start, tp_fused)
    return lm_head_logprobs_ref(x, w, labels, temperature, tp_group, vocab_start)


# --------------------------------------------------------------------------- fused sampling head


def new_sampling_rng(seed: int, device) -> torch.Tensor:
    """State of the fused sampling head: ``[seed, step counter]`` as two 64-bit words on ``device``.
    Every call of :func:`lm_head_sample` advances the counter by one (on the device, so a captured CUDA
    graph draws fresh noise at every replay)."""
    return torch.tensor([int(seed) & 0x7FFFFFFFFFFFFFFF, 0], dtype=torch.int64, device=device)


def lm_head_sample_ref(x, w, temperature, rng_state):
    """PyTorch statement of the fused head: Gumbel-max over ``x @ w.T / temperature`` (argmax where the
    temperature is not positive) and the token's log-probability under the unfiltered distribution."""
    logits = x.float() @ w.float().t()
    t = temperature.float()
    noisy = t > 0
    scaled = logits / torch.where(noisy, t, torch.ones_like(t))[:, None]
    g = torch.Generator(device="cpu").manual_seed(int(rng_state[0]) * 1000003 + int(rng_state[1]))
    u = torch.rand(scaled.shape, generator=g).clamp_(1e-10, 1 - 1e-7).to(scaled.device)
    gumbel = -torch.log(-torch.log(u))
    tokens = torch.where(noisy[:, None], scaled + gumbel, scaled).argmax(-1)
    logp = torch.log_softmax(scaled, -1).gather(1, tokens[:, None]).squeeze(1)
    rng_state[1] += 1
    return tokens.to(torch.int32), logp


def lm_head_sample(x: torch.Tensor, w: torch.Tensor, temperature: torch.Tensor, rng_state: torch.Tensor):
    """Draws ``tokens[b] ~ softmax(x[b] @ w.T / temperature[b])`` inside the LM-head GEMM's epilogue (the
    ``[B, V]`` logits are never written) and returns ``(tokens int32 [B], logprobs f32 [B])``; rows with
    ``temperature <= 0`` take the argmax. Top-k / top-p filtering needs the whole row and goes through
    ``rollout_ops.sample`` on materialised logits instead. The inference servers the reference drives
    sample on materialised logits (areal/engine/sglang_remote.py:43-127 ``sampling_params``)."""
    if not (_lib.use_cuda_kernels(x, w) and x.dtype == torch.bfloat16 and x.shape[1] % 8 == 0):
        return lm_head_sample_ref(x, w, temperature, rng_state)
    B, H = x.shape
    V = w.shape[0]
    lib = _lib.kernels()
    lib.b200_lm_head_sample_nsplit.restype = ctypes.c_int
    nsplit = lib.b200_lm_head_sample_nsplit(ctypes.c_int(B), ctypes.c_int(V))
    partials = torch.empty((nsplit, B, 4), dtype=torch.float32, device=x.device)
    part_idx = torch.empty((nsplit, B), dtype=torch.int32, device=x.device)
    tokens = torch.empty(B, dtype=torch.int32, device=x.device)
    logps = torch.empty(B, dtype=torch.float32, device=x.device)
    x = x if x.stride(1) == 1 else x.contiguous()
    lib.b200_lm_head_sample.restype = ctypes.c_int
    rc = lib.b200_lm_head_sample(_lib.ptr(x), _lib.ptr(w), _lib.ptr(temperature), _lib.ptr(partials),
                                 _lib.ptr(part_idx), _lib.ptr(rng_state), _lib.ptr(tokens), _lib.ptr(logps),
                                 ctypes.c_int(B), ctypes.c_int(V), ctypes.c_int(H), ctypes.c_longlong(x.stride(0)),
                                 ctypes.c_longlong(w.stride(0)), _lib.stream_ptr())
    _lib.check(rc, "b200_lm_head_sample")
    _lib.count_launch(2)
    return tokens, logps
