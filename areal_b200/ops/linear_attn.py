"""Linear-attention ops for hybrid models on packed sequences (``csrc/linear_attn.cu``):
causal depthwise conv1d (+SiLU) with forward and backward kernels, and the gated delta rule /
simple gated linear attention recurrences. The recurrences run their CUDA kernel whenever no
gradient is needed (rollout, logprob recomputation); under autograd they run the PyTorch
restatement below, which is also the test oracle.

Reference call sites: causal_conv1d_fn and fla ``chunk_gated_delta_rule``
(areal/experimental/models/archon/qwen3_5/model/model.py:244,291), fla ``chunk_simple_gla``
(areal/models/mcore/lightning_attention.py:304).
"""

from __future__ import annotations

import ctypes

import torch

from . import _lib


def _seq_of(cu: torch.Tensor, T: int) -> torch.Tensor:
    lens = (cu[1:] - cu[:-1]).long()
    return torch.repeat_interleave(torch.arange(len(lens), device=cu.device), lens, output_size=T).int()


# --------------------------------------------------------------------------- conv1d


def causal_conv1d_ref(x, w, bias, cu, activation: bool = True):
    """``x [T, C]``, ``w [C, K]``, ``cu`` cumulative sequence lengths; no leakage across sequences."""
    T, C = x.shape
    K = w.shape[1]
    out = torch.zeros(T, C, dtype=torch.float32, device=x.device)
    cu_l = [int(c) for c in cu]
    xf = x.float()
    for s0, s1 in zip(cu_l[:-1], cu_l[1:]):
        seg = xf[s0:s1]
        pad = torch.cat([torch.zeros(K - 1, C, device=x.device), seg], 0)
        acc = sum(pad[j:j + (s1 - s0)] * w[:, j].float() for j in range(K))
        out[s0:s1] = acc
    if bias is not None:
        out = out + bias.float()
    if activation:
        out = torch.nn.functional.silu(out)
    return out.to(x.dtype)


class _Conv1d(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias, cu, activation):
        T, C = x.shape
        K = w.shape[1]
        x = x.contiguous()
        w32 = w.float().contiguous()
        b32 = bias.float().contiguous() if bias is not None else None
        cu = cu.int().contiguous()
        seq_of = _seq_of(cu, T)
        y = torch.empty_like(x)
        rc = _lib.kernels().b200_causal_conv1d_fwd(_lib.ptr(x), _lib.ptr(w32), _lib.ptr(b32), _lib.ptr(seq_of),
                                                   _lib.ptr(cu), _lib.ptr(y), ctypes.c_int(T), ctypes.c_int(C),
                                                   ctypes.c_int(K), ctypes.c_int(int(activation)), _lib.stream_ptr())
        _lib.check(rc, "b200_causal_conv1d_fwd")
        _lib.count_launch()
        ctx.save_for_backward(x, w32, b32, seq_of, cu)
        ctx.activation, ctx.w_dtype, ctx.has_bias = activation, w.dtype, bias is not None
        ctx.b_dtype = bias.dtype if bias is not None else None
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w32, b32, seq_of, cu = ctx.saved_tensors
        T, C = x.shape
        K = w32.shape[1]
        dy = dy.contiguous()
        dx = torch.empty_like(x)
        dw = torch.zeros_like(w32)
        db = torch.zeros(C, dtype=torch.float32, device=x.device) if ctx.has_bias else None
        rc = _lib.kernels().b200_causal_conv1d_bwd(_lib.ptr(x), _lib.ptr(dy), _lib.ptr(w32), _lib.ptr(b32),
                                                   _lib.ptr(seq_of), _lib.ptr(cu), _lib.ptr(dx), _lib.ptr(dw), _lib.ptr(db),
                                                   ctypes.c_int(T), ctypes.c_int(C), ctypes.c_int(K),
                                                   ctypes.c_int(int(ctx.activation)), _lib.stream_ptr())
        _lib.check(rc, "b200_causal_conv1d_bwd")
        _lib.count_launch()
        return dx, dw.to(ctx.w_dtype), (db.to(ctx.b_dtype) if db is not None else None), None, None


def causal_conv1d(x, w, bias, cu, activation: bool = True):
    if _lib.use_cuda_kernels(x) and x.dtype == torch.bfloat16 and w.shape[1] <= 7:
        return _Conv1d.apply(x, w, bias, cu, activation)
    return causal_conv1d_ref(x, w, bias, cu, activation)


# --------------------------------------------------------------------------- recurrences


def linear_attn_ref(q, k, v, a, b, cu, scale: float, mode: str):
    """fp32 recurrence. ``q, k [T, H, DK]``, ``v [T, H, DV]``, decay ``a [T, H]`` in (0, 1],
    ``b [T, H]`` (delta rule write strength; ignored for ``simple_gla``)."""
    T, H, DK = q.shape
    DV = v.shape[2]
    out = []
    cu_l = [int(c) for c in cu]
    qf, kf, vf = q.float(), k.float(), v.float()
    for s0, s1 in zip(cu_l[:-1], cu_l[1:]):
        S = torch.zeros(H, DK, DV, dtype=torch.float32, device=q.device)
        for t in range(s0, s1):
            S = S * a[t].float()[:, None, None]
            kt, vt = kf[t], vf[t]
            if mode == "gated_delta":
                u = torch.einsum("hkv,hk->hv", S, kt)
                S = S + torch.einsum("hk,hv->hkv", kt, b[t].float()[:, None] * (vt - u))
            else:
                S = S + torch.einsum("hk,hv->hkv", kt, vt)
            out.append(torch.einsum("hkv,hk->hv", S, qf[t]) * scale)
    return torch.stack(out).to(q.dtype) if out else torch.zeros_like(v)


def linear_attn(q, k, v, a, b, cu, scale: float | None = None, mode: str = "gated_delta"):
    """``o_t = scale * S_t^T q_t`` with ``S_t = a_t S_{t-1} + k_t v_t^T`` (``simple_gla``) or the gated
    delta rule ``S_t = a_t S_{t-1} + b_t k_t (v_t - (a_t S_{t-1})^T k_t)^T``."""
    if mode not in ("gated_delta", "simple_gla"):
        raise ValueError(f"unknown linear-attention mode {mode!r}")
    T, H, DK = q.shape
    DV = v.shape[2]
    scale = scale if scale is not None else DK ** -0.5
    needs_grad = torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in (q, k, v, a, b))
    if needs_grad or not (_lib.use_cuda_kernels(q, k, v) and q.dtype == torch.bfloat16 and DK in (64, 128) and DV <= 256):
        return linear_attn_ref(q, k, v, a, b, cu, scale, mode)
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    a32 = a.float().contiguous()
    b32 = b.float().contiguous() if b is not None else None
    cu = cu.int().contiguous()
    o = torch.empty_like(v)
    rc = _lib.kernels().b200_linear_attn_fwd(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(a32), _lib.ptr(b32),
                                             _lib.ptr(cu), _lib.ptr(o), None, ctypes.c_int(cu.numel() - 1),
                                             ctypes.c_int(H), ctypes.c_int(DK), ctypes.c_int(DV), ctypes.c_float(scale),
                                             ctypes.c_int(1 if mode == "gated_delta" else 0), _lib.stream_ptr())
    _lib.check(rc, "b200_linear_attn_fwd")
    _lib.count_launch()
    return o
