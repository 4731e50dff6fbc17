"""Ulysses sequence parallelism: tokens are sharded over the sp group everywhere except
inside attention, where an all-to-all trades the token shard for a head shard (every rank
then attends over the FULL packed sequence with ``H/S`` heads) and a second all-to-all trades
it back.

``seq_to_head`` / ``head_to_seq`` are the two differentiable exchanges (each is the other's
backward). On CUDA they run on the symmetric-memory all-to-all of ``SymmComm``-style peer
stores when a fused context is given, else on ``all_to_all_single``; gloo has no all-to-all,
so CPU ranks use an all-gather and keep their part (tests only).

Reference: areal/models/fsdp/ulysses.py:153-284 and
areal/models/transformers/ulyssess_patch.py:36-249 (3 exchanges in, 1 out, ``repeat_kv`` when
there are fewer kv heads than ranks).
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from ..ops.attention import VarlenMeta, varlen_attention


def _a2a_seq_to_head(x: torch.Tensor, group, world: int, rank: int) -> torch.Tensor:
    """``x [t, H, D]`` (local tokens, all heads) → ``[t*S, H/S, D]`` (all tokens, local heads)."""
    t, H, D = x.shape
    hs = H // world
    if x.is_cuda:
        send = x.view(t, world, hs, D).transpose(0, 1).contiguous()  # [S, t, hs, D]: block s goes to rank s
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=group)
        return recv.view(world * t, hs, D)  # source-rank major == token order
    parts = [torch.empty_like(x) for _ in range(world)]
    dist.all_gather(parts, x.contiguous(), group=group)
    return torch.cat([p[:, rank * hs:(rank + 1) * hs] for p in parts], 0).contiguous()


def _a2a_head_to_seq(x: torch.Tensor, group, world: int, rank: int) -> torch.Tensor:
    """``x [t*S, H/S, D]`` → ``[t, H, D]``."""
    T, hs, D = x.shape
    t = T // world
    if x.is_cuda:
        send = x.contiguous().view(world, t, hs, D)  # block s = tokens of rank s
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=group)  # recv[s] = my tokens, heads of rank s
        return recv.permute(1, 0, 2, 3).reshape(t, world * hs, D).contiguous()
    parts = [torch.empty_like(x) for _ in range(world)]
    dist.all_gather(parts, x.contiguous(), group=group)
    return torch.cat([p[rank * t:(rank + 1) * t] for p in parts], 1).contiguous()


class _SeqToHead(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, world, rank):
        ctx.args = (group, world, rank)
        return _a2a_seq_to_head(x, group, world, rank)

    @staticmethod
    def backward(ctx, dy):
        return _a2a_head_to_seq(dy, *ctx.args), None, None, None


class _HeadToSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, world, rank):
        ctx.args = (group, world, rank)
        return _a2a_head_to_seq(x, group, world, rank)

    @staticmethod
    def backward(ctx, dy):
        return _a2a_seq_to_head(dy, *ctx.args), None, None, None


def seq_to_head(x, pctx):
    return _SeqToHead.apply(x, pctx.sp_group, pctx.sp_size, pctx.sp_rank)


def head_to_seq(x, pctx):
    return _HeadToSeq.apply(x, pctx.sp_group, pctx.sp_size, pctx.sp_rank)


# --------------------------------------------------------------------------- fused projection


def qkv_rank_major_rows(n_q: int, n_kv: int, head_dim: int, sp: int, device) -> torch.Tensor:
    """Row order of the fused ``[q | k | v]`` projection weight that groups, for every sp rank r,
    ``[q heads of r | k heads of r | v heads of r]``: with it the column block r of the projection
    output is exactly what rank r needs after the exchange."""
    qs, ks = n_q * head_dim, n_kv * head_dim
    q = torch.arange(qs, device=device).view(sp, -1)
    k = (qs + torch.arange(ks, device=device)).view(sp, -1)
    v = (qs + ks + torch.arange(ks, device=device)).view(sp, -1)
    return torch.cat([q, k, v], 1).reshape(-1)


class _FusedQKVSeqToHead(torch.autograd.Function):
    """``seq_to_head(x @ w.T)`` in one kernel: the projection's epilogue stores every rank's head block
    straight into that rank's buffer over NVLink (``fused_linear.gemm_all_to_all``). Backward: the
    reverse exchange (NCCL all-to-all), then the two GEMMs; the weight gradient is scattered back to
    the parameter's own row order (into ``main_grad`` when present)."""

    @staticmethod
    def forward(ctx, x, w, perm, fctx, group, world, rank):
        from . import fused_linear as FL

        w_perm = w.index_select(0, perm)
        y = FL.gemm_all_to_all(fctx, x, w_perm)  # [t * S, N / S]
        ctx.save_for_backward(x, w, w_perm, perm)
        ctx.args = (group, world, rank)
        return y

    @staticmethod
    def backward(ctx, dy):
        from ..ops.gemm import gemm

        x, w, w_perm, perm = ctx.saved_tensors
        group, world, rank = ctx.args
        T, n_loc = dy.shape
        t = T // world
        # [S, t, n_loc] blocks: block s holds the tokens of rank s → send back, receive my tokens' columns of every rank
        send = dy.contiguous().view(world, t, n_loc)
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=group)
        g = recv.permute(1, 0, 2).reshape(t, world * n_loc).contiguous()  # columns in rank-major (w_perm) order
        dx = gemm(g, w_perm, b_mn=True, out_dtype=x.dtype) if ctx.needs_input_grad[0] else None
        dw = None
        if ctx.needs_input_grad[1]:
            dwp = gemm(g, x, a_mn=True, b_mn=True, out_dtype=torch.float32)
            main = getattr(w, "main_grad", None)
            if main is not None:
                main.index_add_(0, perm, dwp)
            else:
                dw = torch.zeros_like(w, dtype=torch.float32).index_add_(0, perm, dwp).to(w.dtype)
        return dx, dw, None, None, None, None, None


def fused_qkv_seq_to_head(x, w, pctx, n_q: int, n_kv: int, head_dim: int):
    """Projection + exchange; returns ``[T_full, (n_q + 2 n_kv) / S * head_dim]`` laid out as
    ``[q_r | k_r | v_r]`` for this rank, or None when the fused kernel does not apply."""
    f = pctx.sp_fused
    S = pctx.sp_size
    if f is None or not f.cuda or not x.is_cuda or x.dtype != torch.bfloat16 or n_kv % S or n_q % S:
        return None
    N = w.shape[0]
    if S * x.shape[0] * (N // S) * 2 > f.max_stage_bytes or (N // S) % 64:
        return None
    key = (n_q, n_kv, head_dim, S, x.device)
    perm = pctx.extras.setdefault("qkv_perm", {}).get(key)
    if perm is None:
        perm = pctx.extras["qkv_perm"][key] = qkv_rank_major_rows(n_q, n_kv, head_dim, S, x.device)
    return _FusedQKVSeqToHead.apply(x, w, perm, f, pctx.sp_group, S, pctx.sp_rank)


class _FusedHeadToSeqProj(torch.autograd.Function):
    """``head_to_seq(a) @ w.T`` through ``fused_linear.all_to_all_gemm`` (the exchange rides inside the
    projection's K loop). Backward: ``dA = dy @ w`` for this rank's tokens and all heads, sent back with
    the reverse exchange (NCCL all-to-all); the weight gradient is one GEMM per received chunk, written
    into its column block (of ``main_grad`` when present)."""

    @staticmethod
    def forward(ctx, a, w, fctx, group, world):
        from . import fused_linear as FL

        y, chunks = FL.all_to_all_gemm(fctx, a, w, return_chunks=True)
        if chunks is None:  # shapes the kernel does not take: the exchange ran unfused
            M = a.shape[0] // world
            send = a.contiguous().view(world, M, a.shape[1])
            chunks = torch.empty_like(send)
            dist.all_to_all_single(chunks, send, group=group)
        ctx.save_for_backward(chunks, w)
        ctx.args = (group, world)
        return y

    @staticmethod
    def backward(ctx, dy):
        from ..ops.gemm import gemm

        chunks, w = ctx.saved_tensors  # [S, M, Kc]
        group, world = ctx.args
        S, M, Kc = chunks.shape
        dy = dy.contiguous()
        da = None
        if ctx.needs_input_grad[0]:
            g = gemm(dy, w, b_mn=True, out_dtype=dy.dtype)  # [M, S * Kc]: my tokens, every rank's heads
            send = g.view(M, S, Kc).permute(1, 0, 2).contiguous()
            recv = torch.empty_like(send)
            dist.all_to_all_single(recv, send, group=group)
            da = recv.view(S * M, Kc)
        dw = None
        if ctx.needs_input_grad[1]:
            main = getattr(w, "main_grad", None)
            acc = main if main is not None else torch.zeros(w.shape, dtype=torch.float32, device=w.device)
            for s_ in range(S):
                gemm(dy, chunks[s_], a_mn=True, b_mn=True, out=acc[:, s_ * Kc:(s_ + 1) * Kc], accumulate=True)
            dw = None if main is not None else acc.to(w.dtype)
        return da, dw, None, None, None


def fused_head_to_seq_proj(a, w, pctx):
    """``a [T_full, heads_local * D]`` → ``[T_full / S, hidden]``; None when the fused kernel does not apply."""
    f = pctx.sp_fused
    S = pctx.sp_size
    if f is None or not f.cuda or not a.is_cuda or a.dtype != torch.bfloat16 or a.shape[0] % S or a.shape[1] % 64 \
            or a.numel() * 2 > f.max_stage_bytes:
        return None
    return _FusedHeadToSeqProj.apply(a, w, f, pctx.sp_group, S)


def ulysses_attention(pctx, inner=None):
    """Returns an ``attn_fn(q, k, v, meta)`` for token-sharded inputs: ``meta`` describes the FULL
    packed sequence (all sp ranks' tokens concatenated in rank order)."""
    inner = inner or varlen_attention
    S = pctx.sp_size

    def attn(q, k, v, meta: VarlenMeta):
        Hkv = k.shape[1]
        if Hkv % S:
            # fewer kv heads than ranks: replicate them so each rank owns whole heads
            assert S % Hkv == 0, f"kv heads {Hkv} vs sp {S}"
            rep = S // Hkv
            k = k.repeat_interleave(rep, 1)
            v = v.repeat_interleave(rep, 1)
        qf, kf, vf = seq_to_head(q, pctx), seq_to_head(k, pctx), seq_to_head(v, pctx)
        out = inner(qf, kf, vf, meta)
        return head_to_seq(out, pctx)

    attn.is_ulysses = True
    return attn
