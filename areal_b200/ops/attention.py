"""Varlen packed causal attention (GQA) on the tcgen05 kernels
(``csrc/attn_fwd.cu`` / ``csrc/attn_bwd.cu``) with a PyTorch fp32 reference.

Inputs are packed: ``q [T, Hq, D]``, ``k/v [T, Hkv, D]`` and ``cu_seqlens [B+1]``
(int32), the same contract as flash-attn's ``flash_attn_varlen_func`` that the
reference calls (areal/experimental/models/archon/attention/varlen.py:19-116).
The work lists (one record per 128-row tile) are built on the host from
``cu_seqlens``, which the packer already has on the CPU.
"""

from __future__ import annotations

import ctypes
import math

import numpy as np
import torch

from . import _lib

_QT = 128
_KT = 64
_BT = 128


class VarlenMeta:
    """Host-built tile tables for one packed batch (reused by every layer)."""

    def __init__(self, cu_seqlens_cpu, device):
        cu = np.asarray(cu_seqlens_cpu, dtype=np.int64)
        self.cu_cpu = cu
        self.total = int(cu[-1])
        self.max_seqlen = int((cu[1:] - cu[:-1]).max()) if len(cu) > 1 else 0
        fwd, bwd = [], []
        for b in range(len(cu) - 1):
            s, e = int(cu[b]), int(cu[b + 1])
            L = e - s
            for q0 in range(0, L, _QT):
                ql = min(_QT, L - q0)
                fwd.append((s + q0, ql, s, min(L, q0 + _QT), q0, 0, 0, 0))
            for k0 in range(0, L, _BT):
                bwd.append((s + k0, min(_BT, L - k0), k0, s, L, 0, 0, 0))
        # longest-running tiles first
        fwd.sort(key=lambda t: -t[3])
        bwd.sort(key=lambda t: -(t[4] - t[2]))
        self.n_fwd = len(fwd)
        self.n_bwd = len(bwd)
        self.fwd_tiles = torch.tensor(fwd, dtype=torch.int32).reshape(-1, 8).to(device)
        self.bwd_tiles = torch.tensor(bwd, dtype=torch.int32).reshape(-1, 8).to(device)
        self.cu_seqlens = torch.tensor(cu, dtype=torch.int32).to(device)


def attention_ref(q, k, v, cu_seqlens, scale=None):
    """fp32 masked-softmax reference, one sequence at a time."""
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    out = torch.empty((T, Hq, D), dtype=torch.float32, device=q.device)
    cu = [int(x) for x in cu_seqlens]
    g = Hq // Hkv
    for b in range(len(cu) - 1):
        s, e = cu[b], cu[b + 1]
        if e == s:
            continue
        qs = q[s:e].float().transpose(0, 1)  # [Hq, L, D]
        ks = k[s:e].float().transpose(0, 1).repeat_interleave(g, dim=0)
        vs = v[s:e].float().transpose(0, 1).repeat_interleave(g, dim=0)
        att = qs @ ks.transpose(1, 2) * scale
        L = e - s
        mask = torch.ones(L, L, dtype=torch.bool, device=q.device).tril()
        att = att.masked_fill(~mask, float("-inf")).softmax(-1)
        out[s:e] = (att @ vs).transpose(0, 1)
    return out.to(q.dtype)


def attention_sdpa(q, k, v, cu_seqlens, scale=None):
    """Per-sequence ``scaled_dot_product_attention`` (PyTorch's fused kernels: no ``L x L`` score tensor): the
    general path for head widths the tcgen05 kernels do not cover once sequences are too long for
    :func:`attention_ref`'s fp32 scores. Differentiable; grouped-query heads are expanded by view."""
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    g = Hq // Hkv
    outs = []
    cu = [int(x) for x in cu_seqlens]
    for s, e in zip(cu[:-1], cu[1:]):
        if e == s:
            continue
        qs = q[s:e].transpose(0, 1).unsqueeze(0)                                   # [1, Hq, L, D]
        ks = k[s:e].transpose(0, 1).repeat_interleave(g, dim=0).unsqueeze(0) if g > 1 else k[s:e].transpose(0, 1).unsqueeze(0)
        vs = v[s:e].transpose(0, 1).repeat_interleave(g, dim=0).unsqueeze(0) if g > 1 else v[s:e].transpose(0, 1).unsqueeze(0)
        o = torch.nn.functional.scaled_dot_product_attention(qs, ks, vs, is_causal=True, scale=scale)
        outs.append(o.squeeze(0).transpose(0, 1))
    return torch.cat(outs, 0) if outs else torch.zeros_like(q)


# above this many bytes of fp32 scores for one sequence the general path switches to `attention_sdpa`
_REF_SCORE_BYTES = 1 << 30


def _fwd_cuda(q, k, v, meta: VarlenMeta, scale):
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    assert D == 128, "the sm_100a attention kernels are specialised for head_dim 128"
    q = q if q.is_contiguous() else q.contiguous()
    assert k.stride(2) == 1 and k.stride(1) == D and v.stride(2) == 1 and v.stride(1) == D
    o = torch.empty_like(q)
    lse = torch.empty((Hq, T), dtype=torch.float32, device=q.device)
    fn = _lib.kernels().b200_attn_fwd
    fn.restype = ctypes.c_int
    rc = fn(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(o), _lib.ptr(lse),
            _lib.ptr(meta.fwd_tiles), ctypes.c_int(meta.n_fwd), ctypes.c_int(T),
            ctypes.c_int(Hq), ctypes.c_int(Hkv), ctypes.c_longlong(q.stride(0)),
            ctypes.c_longlong(k.stride(0)), ctypes.c_longlong(v.stride(0)),
            ctypes.c_float(scale), _lib.stream_ptr())
    _lib.check(rc, "b200_attn_fwd")
    _lib.count_launch()
    return o, lse


def _bwd_cuda(q, k, v, o, do, lse, meta: VarlenMeta, scale, dk_out=None, dv_out=None):
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    do = do if do.is_contiguous() else do.contiguous()
    dq_acc = torch.zeros((T, Hq, D), dtype=torch.float32, device=q.device)
    delta = torch.empty((Hq, T), dtype=torch.float32, device=q.device)
    dq = torch.empty_like(q)
    dk = dk_out if dk_out is not None else torch.empty((T, Hkv, D), dtype=q.dtype, device=q.device)
    dv = dv_out if dv_out is not None else torch.empty((T, Hkv, D), dtype=q.dtype, device=q.device)
    fn = _lib.kernels().b200_attn_bwd
    fn.restype = ctypes.c_int
    rc = fn(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(o), _lib.ptr(do), _lib.ptr(lse),
            _lib.ptr(delta), _lib.ptr(dq_acc), _lib.ptr(dq), _lib.ptr(dk), _lib.ptr(dv),
            _lib.ptr(meta.bwd_tiles), ctypes.c_int(meta.n_bwd), ctypes.c_int(T),
            ctypes.c_int(Hq), ctypes.c_int(Hkv), ctypes.c_longlong(k.stride(0)),
            ctypes.c_longlong(v.stride(0)), ctypes.c_longlong(dk.stride(0)),
            ctypes.c_longlong(dv.stride(0)), ctypes.c_float(scale), _lib.stream_ptr())
    _lib.check(rc, "b200_attn_bwd")
    _lib.count_launch(3)
    return dq, dk, dv


class _VarlenAttn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, meta, scale):
        o, lse = _fwd_cuda(q, k, v, meta, scale)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.meta = meta
        ctx.scale = scale
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse = ctx.saved_tensors
        from ..utils.determinism import deterministic_mode

        if deterministic_mode():
            # the kernel accumulates dQ tiles with floating-point atomics (arrival order): bit-stable runs
            # recompute the backward through the PyTorch formulation instead
            with torch.enable_grad():
                qf, kf, vf = (t.detach().float().requires_grad_() for t in (q, k, v))
                of = attention_ref(qf, kf, vf, ctx.meta.cu_cpu, ctx.scale)
                dq, dk, dv = torch.autograd.grad(of, (qf, kf, vf), do.float())
            return dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype), None, None
        dq, dk, dv = _bwd_cuda(q, k, v, o, do, lse, ctx.meta, ctx.scale)
        return dq, dk, dv, None, None


def varlen_attention(q, k, v, meta: VarlenMeta, scale: float | None = None):
    """Causal attention over packed sequences. ``k``/``v`` may be strided views of
    a fused qkv buffer (their token pitch is passed to the TMA descriptor)."""
    D = q.shape[-1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if _lib.use_cuda_kernels(q, k, v) and q.dtype == torch.bfloat16 and D == 128:
        return _VarlenAttn.apply(q, k, v, meta, scale)
    if q.is_cuda:
        _lib.count_fallback(f"varlen_attention[D={D},{str(q.dtype).replace('torch.', '')}]")
        cu = meta.cu_cpu
        longest = max((int(b) - int(a) for a, b in zip(cu[:-1], cu[1:])), default=0)
        if longest * longest * q.shape[1] * 4 > _REF_SCORE_BYTES:
            return attention_sdpa(q, k, v, cu, scale)
    return attention_ref(q, k, v, meta.cu_cpu, scale)
