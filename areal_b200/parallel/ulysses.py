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

    return attn
