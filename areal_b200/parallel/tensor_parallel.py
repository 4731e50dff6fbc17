"""Tensor-parallel linears with sequence-parallel activations.

Between transformer blocks the packed token dimension is sharded over the tp group
(``[T/P, H]`` per rank). A column-parallel linear (qkv, gate_up) is *all-gather → GEMM*,
a row-parallel linear (o_proj, down_proj) is *GEMM → reduce-scatter*; each backward is the
other pattern, so both directions of both layers run on the two fused kernels of
``fused_linear`` (tile-wise NVLink transfers inside the GEMM) when CUDA is available, and on
``torch.distributed`` collectives otherwise (CPU / gloo, also the oracle of the tests).

Reference plan: areal/engine/fsdp_utils/parallel.py:219-367 (DTensor colwise / rowwise with
``Shard(1)`` activations) and Megatron's Column/RowParallelLinear with sequence parallelism.
Weight gradients are written into ``param.main_grad`` (fp32) when the engine provides one.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from ..ops.gemm import gemm
from . import fused_linear as FL


def _use_kernel(t: torch.Tensor) -> bool:
    return t.is_cuda and t.dtype == torch.bfloat16


def _xwt(x, w):
    return gemm(x, w, out_dtype=x.dtype) if _use_kernel(x) else x @ w.t()


def _wgrad(dy, x, w):
    """``dy.T @ x`` into ``w.main_grad`` when present; returns the gradient otherwise."""
    main = getattr(w, "main_grad", None)
    if _use_kernel(dy):
        if main is not None:
            gemm(dy, x, a_mn=True, b_mn=True, out=main, accumulate=True)
            return None
        return gemm(dy, x, a_mn=True, b_mn=True, out_dtype=w.dtype)
    g = dy.t() @ x
    if main is not None:
        main.add_(g.to(main.dtype))
        return None
    return g.to(w.dtype)


def all_gather_rows(fctx, x):
    return FL.ctx_all_gather(fctx, x) if fctx.world > 1 else x


def reduce_scatter_rows(fctx, x):
    """Sum over the group, rank r keeps rows ``[r*M/P, (r+1)*M/P)``."""
    if fctx.world == 1:
        return x
    n = x.shape[0] // fctx.world
    if x.is_cuda:
        out = torch.empty((n,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.reduce_scatter_tensor(out, x.contiguous(), group=fctx.group)
        return out
    y = x.clone()
    dist.all_reduce(y, group=fctx.group)
    return y[fctx.rank * n:(fctx.rank + 1) * n].contiguous()


class _ColumnParallel(torch.autograd.Function):
    """``all_gather_rows(x) @ w.T``: ``x [T/P, K]`` (token shard), ``w [N/P, K]`` → ``[T, N/P]``."""

    @staticmethod
    def forward(ctx, x, w, bias, fctx):
        y = FL.all_gather_gemm(fctx, x, w)
        if bias is not None:
            y = y + bias
        ctx.save_for_backward(x, w)
        ctx.fctx = fctx
        ctx.has_bias = bias is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        fctx = ctx.fctx
        dy = dy.contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            # reduce_scatter(dy @ w): the fused kernel wants the weight as [out, in_shard] = w.T
            dx = FL.gemm_reduce_scatter(fctx, dy, w.t().contiguous())
        if ctx.needs_input_grad[1]:
            dw = _wgrad(dy, all_gather_rows(fctx, x), w)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy.float().sum(0).to(dy.dtype)
        return dx, dw, db, None


class _RowParallel(torch.autograd.Function):
    """``reduce_scatter_rows(x @ w.T)``: ``x [T, K/P]``, ``w [N, K/P]`` → ``[T/P, N]``."""

    @staticmethod
    def forward(ctx, x, w, fctx):
        ctx.save_for_backward(x, w)
        ctx.fctx = fctx
        return FL.gemm_reduce_scatter(fctx, x, w)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        fctx = ctx.fctx
        dy = dy.contiguous()
        # all_gather(dy) @ w, and the gathered rows come back for the weight gradient
        dx, dy_full = FL.all_gather_gemm(fctx, dy, w.t().contiguous(), return_gathered=True)
        dw = _wgrad(dy_full, x, w) if ctx.needs_input_grad[1] else None
        return (dx if ctx.needs_input_grad[0] else None), dw, None


def column_parallel_linear(x, w, fctx, bias=None):
    if fctx is None or fctx.world == 1:
        from ..ops.gemm import linear

        return linear(x, w, bias)
    return _ColumnParallel.apply(x, w, bias, fctx)


def row_parallel_linear(x, w, fctx):
    if fctx is None or fctx.world == 1:
        from ..ops.gemm import linear

        return linear(x, w)
    return _RowParallel.apply(x, w, fctx)


class _GatherSeq(torch.autograd.Function):
    """All-gather of token shards; the backward sums and scatters (every rank produced a
    partial gradient for every token)."""

    @staticmethod
    def forward(ctx, x, fctx):
        ctx.fctx = fctx
        return all_gather_rows(fctx, x)

    @staticmethod
    def backward(ctx, dy):
        return reduce_scatter_rows(ctx.fctx, dy.contiguous()), None


class _ScatterSeqSum(torch.autograd.Function):
    """Reduce-scatter of per-rank partial rows; the backward all-gathers."""

    @staticmethod
    def forward(ctx, x, fctx):
        ctx.fctx = fctx
        return reduce_scatter_rows(fctx, x)

    @staticmethod
    def backward(ctx, dy):
        return all_gather_rows(ctx.fctx, dy.contiguous()), None


class _GatherSeqSlice(torch.autograd.Function):
    """All-gather whose consumers compute the SAME thing on every rank (e.g. a replicated loss):
    the backward keeps this rank's slice, no sum."""

    @staticmethod
    def forward(ctx, x, fctx):
        ctx.fctx = fctx
        return all_gather_rows(fctx, x)

    @staticmethod
    def backward(ctx, dy):
        f = ctx.fctx
        n = dy.shape[0] // f.world
        return dy[f.rank * n:(f.rank + 1) * n].contiguous(), None


def gather_seq(x, fctx):
    return x if (fctx is None or fctx.world == 1) else _GatherSeq.apply(x, fctx)


def scatter_seq_sum(x, fctx):
    return x if (fctx is None or fctx.world == 1) else _ScatterSeqSum.apply(x, fctx)


def gather_seq_replicated(x, fctx):
    return x if (fctx is None or fctx.world == 1) else _GatherSeqSlice.apply(x, fctx)


def vocab_parallel_embedding(ids, embed_shard, fctx):
    """``ids [T]`` (all tokens) with ``embed_shard [V/P, H]`` → token-sharded ``[T/P, H]``: masked
    local lookup, then one reduce-scatter delivers each rank its rows."""
    from ..ops.fused import embedding

    vp = embed_shard.shape[0]
    v0 = fctx.rank * vp
    local = ids - v0
    mask = (local >= 0) & (local < vp)
    part = embedding(torch.where(mask, local, torch.zeros_like(local)), embed_shard)
    part = part * mask.unsqueeze(-1).to(part.dtype)
    return scatter_seq_sum(part, fctx)


# --------------------------------------------------------------------------- weight sharding


# latent attention: the projections out of the bottlenecks (and a plain query projection) are split by head, i.e. by
# contiguous blocks of rows; the projections into the bottlenecks and their norms are replicated
_MLA_BY_HEAD = ("attn.q_b", "attn.kv_b", "attn.q")


def tp_slice(name: str, full: torch.Tensor, cfg, rank: int, size: int) -> torch.Tensor:
    """The tp shard of a (fused) parameter of ``models.qwen``; ``name`` is the parameter's
    attribute path suffix (``embed``, ``attn.qkv``, ``attn.o``, ``mlp.gate_up``, ...)."""
    if size == 1:
        return full
    D = cfg.head_dim
    if name.endswith(("embed", "lm_head") + _MLA_BY_HEAD):
        n = full.shape[0] // size
        return full[rank * n:(rank + 1) * n]
    if name.endswith(("attn.qkv", "attn.qkv_bias")):
        qs, ks = cfg.q_size, cfg.kv_size
        q, k, v = full[:qs], full[qs:qs + ks], full[qs + ks:]
        nq, nk = qs // size, ks // size
        return torch.cat([q[rank * nq:(rank + 1) * nq], k[rank * nk:(rank + 1) * nk], v[rank * nk:(rank + 1) * nk]], 0)
    if name.endswith("attn.o"):
        n = full.shape[1] // size
        return full[:, rank * n:(rank + 1) * n]
    if name.endswith("mlp.gate_up"):
        I = full.shape[0] // 2
        n = I // size
        return torch.cat([full[rank * n:(rank + 1) * n], full[I + rank * n:I + (rank + 1) * n]], 0)
    if name.endswith("mlp.down"):
        n = full.shape[1] // size
        return full[:, rank * n:(rank + 1) * n]
    return full  # norms, score head, router: replicated


def tp_unslice(name: str, shards: list[torch.Tensor], cfg) -> torch.Tensor:
    """Inverse of :func:`tp_slice` given every rank's shard."""
    size = len(shards)
    if size == 1:
        return shards[0]
    if ".lora_" in name:
        d = lora_tp_dim(name)
        return shards[0] if d is None else torch.cat(shards, d)
    if name.endswith(("embed", "lm_head") + _MLA_BY_HEAD):
        return torch.cat(shards, 0)
    if name.endswith(("attn.qkv", "attn.qkv_bias")):
        nq, nk = cfg.q_size // size, cfg.kv_size // size
        return torch.cat([s[:nq] for s in shards] + [s[nq:nq + nk] for s in shards] + [s[nq + nk:] for s in shards], 0)
    if name.endswith(("attn.o", "mlp.down")):
        return torch.cat(shards, 1)
    if name.endswith("mlp.gate_up"):
        n = shards[0].shape[0] // 2
        return torch.cat([s[:n] for s in shards] + [s[n:] for s in shards], 0)
    return shards[0]


def tp_slice_lora_b(name: str) -> bool:
    """Whether the ``lora_B`` factor with this parameter name is split over the tensor-parallel group (the adapters
    of column-parallel projections: B follows the output rows; those of row-parallel projections keep B whole and
    split A along the input)."""
    return ".lora_qkv." in name or ".lora_gate_up." in name


def expert_slice(name: str, full: torch.Tensor, rank: int, size: int) -> torch.Tensor:
    """Slice ``rank`` of ``size`` of stacked expert weights along the expert width: ``gate_up [E, 2I, H]`` keeps
    rows ``[rank * I/size, (rank + 1) * I/size)`` of the gate half and of the up half, ``down [E, H, I]`` the
    matching columns."""
    if name.endswith("gate_up"):
        I = full.shape[1] // 2
        n = I // size
        return torch.cat((full[:, rank * n:(rank + 1) * n], full[:, I + rank * n: I + (rank + 1) * n]), 1)
    n = full.shape[2] // size
    return full[:, :, rank * n:(rank + 1) * n]


def expert_unslice(name: str, shards: list[torch.Tensor]) -> torch.Tensor:
    """Inverse of :func:`expert_slice` over all ranks' shards."""
    if name.endswith("gate_up"):
        n = shards[0].shape[1] // 2
        return torch.cat([s[:, :n] for s in shards] + [s[:, n:] for s in shards], 1)
    return torch.cat(shards, 2)


def lora_tp_dim(name: str) -> int | None:
    """Dimension along which a low-rank adapter factor is split over the tensor-parallel group: ``B`` of a
    column-parallel projection by rows, ``A`` of a row-parallel projection by columns; ``None``: replicated."""
    if (".lora_qkv." in name or ".lora_gate_up." in name) and ".lora_B." in name:
        return 0
    if (".lora_o." in name or ".lora_down." in name) and name.endswith("lora_A"):
        return 1
    return None


def is_tp_replicated(name: str) -> bool:
    if ".lora_" in name:
        return lora_tp_dim(name) is None
    return not name.endswith(("embed", "lm_head", "attn.qkv", "attn.qkv_bias", "attn.o", "mlp.gate_up", "mlp.down")
                             + _MLA_BY_HEAD)
