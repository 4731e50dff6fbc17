"""RMSNorm (+residual), q/k-norm + RoPE and SwiGLU: autograd wrappers over the
kernels in ``csrc/norm_rope_swiglu.cu`` plus fp32 PyTorch references (which are
the CPU path and the oracles of the GPU tests).

Semantics follow the reference models: RMSNorm is computed in fp32 and cast
(areal/experimental/models/archon/qwen3/model/model.py:75-101), RoPE is the
``rotate_half`` form (qwen2/model/rope.py), the MLP is ``w2(silu(w1 x) * w3 x)``.
"""

from __future__ import annotations

import ctypes

import torch

from . import _lib

# --------------------------------------------------------------------------- RMSNorm


def rmsnorm_ref(x, w, eps, residual=None):
    h = x.float() + residual.float() if residual is not None else x.float()
    if residual is not None:
        h = h.to(x.dtype).float()
    y = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + eps) * w.float()
    if residual is not None:
        return y.to(x.dtype), h.to(x.dtype)
    return y.to(x.dtype)


class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps, residual):
        H = x.shape[-1]
        x2 = x.reshape(-1, H)
        x2 = x2 if x2.is_contiguous() else x2.contiguous()
        T = x2.shape[0]
        y = torch.empty_like(x2)
        rstd = torch.empty(T, dtype=torch.float32, device=x.device)
        lib = _lib.kernels()
        lib.b200_rmsnorm_fwd.restype = ctypes.c_int
        if residual is not None:
            r2 = residual.reshape(-1, H)
            r2 = r2 if r2.is_contiguous() else r2.contiguous()
            h = torch.empty_like(x2)
        else:
            r2, h = None, None
        rc = lib.b200_rmsnorm_fwd(_lib.ptr(x2), _lib.ptr(r2), _lib.ptr(w), _lib.ptr(y), _lib.ptr(h),
                                  _lib.ptr(rstd), ctypes.c_int(T), ctypes.c_int(H),
                                  ctypes.c_float(eps), _lib.stream_ptr())
        _lib.check(rc, "b200_rmsnorm_fwd")
        _lib.count_launch()
        ctx.save_for_backward(h if h is not None else x2, w, rstd)
        ctx.has_res = residual is not None
        ctx.shape = x.shape
        if residual is not None:
            return y.view(x.shape), h.view(x.shape)
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy, dh=None):
        xin, w, rstd = ctx.saved_tensors
        T, H = xin.shape
        dy2 = dy.reshape(T, H)
        dy2 = dy2 if dy2.is_contiguous() else dy2.contiguous()
        dres = None
        if ctx.has_res and dh is not None:
            dres = dh.reshape(T, H)
            dres = dres if dres.is_contiguous() else dres.contiguous()
        lib = _lib.kernels()
        lib.b200_rmsnorm_bwd_blocks.restype = ctypes.c_int
        nb = lib.b200_rmsnorm_bwd_blocks(ctypes.c_int(T))
        partial = torch.empty((nb, H), dtype=torch.float32, device=xin.device)
        dw = torch.empty(H, dtype=torch.float32, device=xin.device)
        dx = torch.empty_like(xin)
        lib.b200_rmsnorm_bwd.restype = ctypes.c_int
        rc = lib.b200_rmsnorm_bwd(_lib.ptr(dy2), _lib.ptr(xin), _lib.ptr(w), _lib.ptr(rstd),
                                  _lib.ptr(dres), _lib.ptr(dx), _lib.ptr(partial), _lib.ptr(dw),
                                  ctypes.c_int(0), ctypes.c_int(T), ctypes.c_int(H),
                                  _lib.stream_ptr())
        _lib.check(rc, "b200_rmsnorm_bwd")
        _lib.count_launch(2)
        dxv = dx.view(ctx.shape)
        return dxv, dw.to(w.dtype), None, (dxv if ctx.has_res else None)


def rmsnorm(x, w, eps: float = 1e-6, residual=None):
    """``y = rmsnorm(x (+ residual)) * w``. With ``residual`` returns ``(y, x + residual)``."""
    if _lib.use_cuda_kernels(x) and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0 \
            and x.shape[-1] <= 8192:
        return _RMSNorm.apply(x, w, eps, residual)
    return rmsnorm_ref(x, w, eps, residual)


# --------------------------------------------------------------------------- RoPE


def rope_inv_freq(dim: int, theta: float, scaling: dict | None, device) -> tuple[torch.Tensor, float]:
    """Inverse frequencies of the rotary table and the factor applied to cos / sin.

    ``scaling`` follows the Hugging Face ``rope_scaling`` dictionaries: ``linear`` divides every frequency by
    ``factor``; ``llama3`` keeps wavelengths below ``original_max / high_freq_factor``, divides those above
    ``original_max / low_freq_factor`` by ``factor`` and blends in between; ``yarn`` blends interpolated and
    extrapolated frequencies with a linear ramp over the dimensions between the ``beta_fast`` / ``beta_slow``
    rotations and scales the table by ``0.1 * ln(factor) + 1`` (or ``attention_factor``)."""
    import math

    inv = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float32, device=device) / dim))
    kind = (scaling or {}).get("rope_type", "default")
    if kind == "default":
        return inv, 1.0
    factor = float(scaling["factor"])
    if kind == "linear":
        return inv / factor, 1.0
    if kind == "llama3":
        lo, hi = float(scaling.get("low_freq_factor", 1.0)), float(scaling.get("high_freq_factor", 4.0))
        old_len = float(scaling["original_max_position_embeddings"])
        wavelen = 2 * math.pi / inv
        smooth = ((old_len / wavelen - lo) / (hi - lo)).clamp(0.0, 1.0)
        return (1 - smooth) * inv / factor + smooth * inv, 1.0
    if kind == "yarn":
        old_len = float(scaling.get("original_max_position_embeddings") or 0) or None
        if old_len is None:
            raise ValueError("yarn rope scaling needs original_max_position_embeddings")
        fast, slow = float(scaling.get("beta_fast") or 32), float(scaling.get("beta_slow") or 1)

        def correction_dim(rotations):
            return dim * math.log(old_len / (rotations * 2 * math.pi)) / (2 * math.log(theta))

        low, high = correction_dim(fast), correction_dim(slow)
        if scaling.get("truncate", True):
            low, high = math.floor(low), math.ceil(high)
        low, high = max(low, 0), min(high, dim - 1)
        if low == high:
            high += 0.001
        ramp = ((torch.arange(dim // 2, dtype=torch.float32, device=device) - low) / (high - low)).clamp(0, 1)
        extrap = 1 - ramp
        inv = inv / factor * (1 - extrap) + inv * extrap
        att = scaling.get("attention_factor")
        if att is None:
            mscale, mscale_all = scaling.get("mscale"), scaling.get("mscale_all_dim")
            get = lambda sc, m=1.0: 1.0 if sc <= 1 else 0.1 * m * math.log(sc) + 1.0
            att = get(factor, mscale) / get(factor, mscale_all) if mscale and mscale_all else get(factor)
        return inv, float(att)
    raise NotImplementedError(f"rope scaling {kind!r}")


def rope_tables(max_pos: int, dim: int, theta: float, device,
                scaling: dict | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    inv, att = rope_inv_freq(dim, theta, scaling, device)
    t = torch.arange(max_pos, dtype=torch.float32, device=device)
    fr = torch.outer(t, inv)
    return (fr.cos() * att).contiguous(), (fr.sin() * att).contiguous()


def _rot_half(x):
    d = x.shape[-1] // 2
    return torch.cat((-x[..., d:], x[..., :d]), -1)


def qknorm_rope_ref(qkv, qw, kw, cos, sin, pos, Hq, Hkv, D, eps):
    """qkv [T, (Hq+2Hkv)*D] → q [T,Hq,D], k [T,Hkv,D], v view."""
    T = qkv.shape[0]
    q = qkv[:, : Hq * D].reshape(T, Hq, D)
    k = qkv[:, Hq * D: (Hq + Hkv) * D].reshape(T, Hkv, D)
    v = qkv[:, (Hq + Hkv) * D:].reshape(T, Hkv, D)
    if qw is not None:
        q = rmsnorm_ref(q, qw, eps)
        k = rmsnorm_ref(k, kw, eps)
    c = torch.cat((cos[pos.long()], cos[pos.long()]), -1)[:, None, :]
    s = torch.cat((sin[pos.long()], sin[pos.long()]), -1)[:, None, :]
    qo = (q.float() * c + _rot_half(q.float()) * s).to(qkv.dtype)
    ko = (k.float() * c + _rot_half(k.float()) * s).to(qkv.dtype)
    return qo, ko, v


class _QKNormRope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, qw, kw, cos, sin, pos, Hq, Hkv, D, eps):
        T = qkv.shape[0]
        qkv = qkv if qkv.is_contiguous() else qkv.contiguous()
        has_norm = qw is not None
        q = torch.empty((T, Hq, D), dtype=qkv.dtype, device=qkv.device)
        k = torch.empty((T, Hkv, D), dtype=qkv.dtype, device=qkv.device)
        rstd = torch.empty(T * (Hq + Hkv) if has_norm else 1, dtype=torch.float32,
                           device=qkv.device)
        if _lib.checked():
            _check_rope_args("qknorm_rope", qkv, qw, kw, cos, sin, pos, Hq, Hkv, D)
        lib = _lib.kernels()
        lib.b200_qknorm_rope_fwd.restype = ctypes.c_int
        rc = lib.b200_qknorm_rope_fwd(_lib.ptr(qkv), _lib.ptr(qw), _lib.ptr(kw), _lib.ptr(cos),
                                      _lib.ptr(sin), _lib.ptr(pos), _lib.ptr(q), _lib.ptr(k),
                                      _lib.ptr(rstd), ctypes.c_int(T), ctypes.c_int(Hq),
                                      ctypes.c_int(Hkv), ctypes.c_int(D), ctypes.c_float(eps),
                                      ctypes.c_int(int(has_norm)), _lib.stream_ptr())
        _lib.check(rc, "b200_qknorm_rope_fwd")
        _lib.count_launch()
        v = qkv[:, (Hq + Hkv) * D:].view(T, Hkv, D)
        ctx.save_for_backward(qkv, qw, kw, cos, sin, pos, rstd)
        ctx.dims = (T, Hq, Hkv, D, has_norm)
        ctx.mark_non_differentiable()
        return q, k, v

    @staticmethod
    def backward(ctx, dq, dk, dv):
        qkv, qw, kw, cos, sin, pos, rstd = ctx.saved_tensors
        T, Hq, Hkv, D, has_norm = ctx.dims
        dqkv = torch.empty_like(qkv)
        # dv goes straight into the v slot of the fused gradient
        dqkv[:, (Hq + Hkv) * D:].view(T, Hkv, D).copy_(dv)
        dq = dq if dq.is_contiguous() else dq.contiguous()
        dk = dk if dk.is_contiguous() else dk.contiguous()
        dqw = torch.zeros(D, dtype=torch.float32, device=qkv.device)
        dkw = torch.zeros(D, dtype=torch.float32, device=qkv.device)
        lib = _lib.kernels()
        lib.b200_qknorm_rope_bwd.restype = ctypes.c_int
        rc = lib.b200_qknorm_rope_bwd(_lib.ptr(dq), _lib.ptr(dk), _lib.ptr(qkv), _lib.ptr(qw),
                                      _lib.ptr(kw), _lib.ptr(cos), _lib.ptr(sin), _lib.ptr(pos),
                                      _lib.ptr(rstd), _lib.ptr(dqkv), _lib.ptr(dqw), _lib.ptr(dkw),
                                      ctypes.c_int(T), ctypes.c_int(Hq), ctypes.c_int(Hkv),
                                      ctypes.c_int(D), ctypes.c_int(int(has_norm)),
                                      _lib.stream_ptr())
        _lib.check(rc, "b200_qknorm_rope_bwd")
        _lib.count_launch()
        if has_norm:
            return dqkv, dqw.to(qw.dtype), dkw.to(kw.dtype), None, None, None, None, None, None, None
        return dqkv, None, None, None, None, None, None, None, None, None


def _check_rope_args(site, qkv, qw, kw, cos, sin, pos, Hq, Hkv, D):
    T = qkv.shape[0]
    _lib.check_operand(f"{site}.qkv", qkv, torch.bfloat16, (T, (Hq + 2 * Hkv) * D))
    _lib.check_operand(f"{site}.cos", cos, torch.float32, (None, D // 2), align=8)
    _lib.check_operand(f"{site}.sin", sin, torch.float32, tuple(cos.shape), align=8)
    _lib.check_operand(f"{site}.pos", pos, torch.int32, (T,), align=4)
    _lib.check_operand(f"{site}.q_norm", qw, torch.bfloat16, (D,), align=4)
    _lib.check_operand(f"{site}.k_norm", kw, torch.bfloat16, (D,), align=4)
    _lib.check_index(f"{site}.pos", pos, cos.shape[0])


def qknorm_rope(qkv, qw, kw, cos, sin, pos, Hq, Hkv, D, eps=1e-6):
    """Splits a fused qkv projection, applies per-head RMSNorm to q and k (when
    ``qw``/``kw`` are given, Qwen3) and rotary embedding; returns ``(q, k, v)``
    with ``v`` a strided view of ``qkv``."""
    if _lib.use_cuda_kernels(qkv) and qkv.dtype == torch.bfloat16 and D == 128:
        return _QKNormRope.apply(qkv, qw, kw, cos, sin, pos, Hq, Hkv, D, eps)
    return qknorm_rope_ref(qkv, qw, kw, cos, sin, pos, Hq, Hkv, D, eps)


@torch.no_grad()
def qknorm_rope_kvwrite(qkv, qw, kw, cos, sin, pos, Hq, Hkv, D, eps, slot_mapping, k_cache, v_cache):
    """Inference form of :func:`qknorm_rope`: returns ``q [T, Hq, D]`` and writes the normalised,
    rotated ``k`` and the raw ``v`` into the paged caches ``[num_blocks, Hkv, block_size, D]`` at
    ``slot_mapping [T]`` (int64, negative = skip) in the same kernel."""
    if not (_lib.use_cuda_kernels(qkv, k_cache) and qkv.dtype == torch.bfloat16 and D == 128 and qkv.is_contiguous()):
        from .rollout_ops import kv_cache_write

        q, k, v = qknorm_rope(qkv, qw, kw, cos, sin, pos, Hq, Hkv, D, eps)
        kv_cache_write(k, v, slot_mapping, k_cache, v_cache)
        return q
    T = qkv.shape[0]
    q = torch.empty((T, Hq, D), dtype=qkv.dtype, device=qkv.device)
    slots = slot_mapping if slot_mapping.dtype == torch.int64 else slot_mapping.to(torch.int64)
    if _lib.checked():
        _check_rope_args("qknorm_rope_kvwrite", qkv, qw, kw, cos, sin, pos, Hq, Hkv, D)
        _lib.check_operand("qknorm_rope_kvwrite.k_cache", k_cache, torch.bfloat16, (None, Hkv, None, D))
        _lib.check_operand("qknorm_rope_kvwrite.v_cache", v_cache, torch.bfloat16, tuple(k_cache.shape))
        _lib.check_index("qknorm_rope_kvwrite.slot_mapping", slots[:T], k_cache.shape[0] * k_cache.shape[2],
                         allow_negative=True)
    rc = _lib.kernels().b200_qknorm_rope_kvwrite(
        _lib.ptr(qkv), _lib.ptr(qw), _lib.ptr(kw), _lib.ptr(cos), _lib.ptr(sin), _lib.ptr(pos), _lib.ptr(q),
        _lib.ptr(slots.contiguous()), _lib.ptr(k_cache), _lib.ptr(v_cache), ctypes.c_int(T), ctypes.c_int(Hq),
        ctypes.c_int(Hkv), ctypes.c_int(D), ctypes.c_int(k_cache.shape[2]), ctypes.c_float(eps),
        ctypes.c_int(int(qw is not None)), _lib.stream_ptr())
    _lib.check(rc, "b200_qknorm_rope_kvwrite")
    _lib.count_launch()
    return q


# --------------------------------------------------------------------------- SwiGLU


def swiglu_ref(gu):
    inter = gu.shape[-1] // 2
    g, u = gu[..., :inter].float(), gu[..., inter:].float()
    return (torch.nn.functional.silu(g) * u).to(gu.dtype)


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        inter = gu.shape[-1] // 2
        g2 = gu.reshape(-1, 2 * inter)
        g2 = g2 if g2.is_contiguous() else g2.contiguous()
        out = torch.empty((g2.shape[0], inter), dtype=gu.dtype, device=gu.device)
        lib = _lib.kernels()
        lib.b200_swiglu_fwd.restype = ctypes.c_int
        rc = lib.b200_swiglu_fwd(_lib.ptr(g2), _lib.ptr(out), ctypes.c_longlong(g2.shape[0]),
                                 ctypes.c_int(inter), _lib.stream_ptr())
        _lib.check(rc, "b200_swiglu_fwd")
        _lib.count_launch()
        ctx.save_for_backward(g2)
        ctx.shape = gu.shape
        return out.view(*gu.shape[:-1], inter)

    @staticmethod
    def backward(ctx, dy):
        (g2,) = ctx.saved_tensors
        inter = g2.shape[1] // 2
        dy2 = dy.reshape(-1, inter)
        dy2 = dy2 if dy2.is_contiguous() else dy2.contiguous()
        dgu = torch.empty_like(g2)
        lib = _lib.kernels()
        lib.b200_swiglu_bwd.restype = ctypes.c_int
        rc = lib.b200_swiglu_bwd(_lib.ptr(dy2), _lib.ptr(g2), _lib.ptr(dgu),
                                 ctypes.c_longlong(g2.shape[0]), ctypes.c_int(inter),
                                 _lib.stream_ptr())
        _lib.check(rc, "b200_swiglu_bwd")
        _lib.count_launch()
        return dgu.view(ctx.shape)


def swiglu(gu):
    """``silu(gu[..., :I]) * gu[..., I:]`` for a fused gate/up projection."""
    if _lib.use_cuda_kernels(gu) and gu.dtype == torch.bfloat16 and (gu.shape[-1] // 2) % 8 == 0:
        return _SwiGLU.apply(gu)
    return swiglu_ref(gu)


# --------------------------------------------------------------------------- embedding


def _embedding_kernel_ok(ids: torch.Tensor, w: torch.Tensor) -> bool:
    return (_lib.use_cuda_kernels(ids, w) and w.dtype == torch.bfloat16 and w.dim() == 2
            and w.shape[1] % 8 == 0 and w.is_contiguous())


def _embedding_fwd(ids: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    if not _embedding_kernel_ok(ids, w):
        if w.is_cuda:
            _lib.count_fallback(f"embedding_fwd[{str(w.dtype).replace('torch.', '')}]")
        return torch.nn.functional.embedding(ids, w)
    flat = ids.reshape(-1).contiguous()
    out = torch.empty((flat.numel(), w.shape[1]), dtype=w.dtype, device=w.device)
    rc = _lib.kernels().b200_embedding_fwd(_lib.ptr(flat), _lib.ptr(w), _lib.ptr(out), ctypes.c_int(flat.numel()),
                                           ctypes.c_int(w.shape[1]), ctypes.c_longlong(w.shape[0]), _lib.stream_ptr())
    _lib.check(rc, "b200_embedding_fwd")
    _lib.count_launch()
    return out.view(*ids.shape, w.shape[1])


class _Embedding(torch.autograd.Function):
    """Embedding lookup whose backward scatter-adds straight into the weight's fp32
    ``main_grad`` (when present) instead of materialising a dense ``[V, H]`` gradient."""

    @staticmethod
    def forward(ctx, ids, w):
        ctx.save_for_backward(ids)
        ctx.w = w
        return _embedding_fwd(ids, w)

    @staticmethod
    def backward(ctx, dy):
        (ids,) = ctx.saved_tensors
        w = ctx.w
        main = getattr(w, "main_grad", None)
        dy2 = dy.reshape(-1, dy.shape[-1])
        # the kernel's atomic adds sum rows of equal id in varying order: under deterministic mode the
        # sorted PyTorch scatter runs instead
        use_kernel = (_embedding_kernel_ok(ids, w) and dy.dtype == torch.bfloat16
                      and not torch.are_deterministic_algorithms_enabled())
        target = main if main is not None else torch.zeros(w.shape, dtype=torch.float32, device=w.device)
        if use_kernel and target.is_contiguous():
            flat = ids.reshape(-1).contiguous()
            rc = _lib.kernels().b200_embedding_bwd(_lib.ptr(flat), _lib.ptr(dy2.contiguous()), _lib.ptr(target),
                                                   ctypes.c_int(flat.numel()), ctypes.c_int(w.shape[1]),
                                                   ctypes.c_longlong(w.shape[0]), _lib.stream_ptr())
            _lib.check(rc, "b200_embedding_bwd")
            _lib.count_launch()
        else:
            if w.is_cuda:
                _lib.count_fallback("embedding_bwd[index_add]")
            target.index_add_(0, ids.reshape(-1), dy2.to(torch.float32))
        return None, (None if main is not None else target.to(w.dtype))


def embedding(ids: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``w[ids]`` for ids in ``[0, V)``; ids outside that range give zero rows on the kernel path."""
    if w.requires_grad and torch.is_grad_enabled():
        return _Embedding.apply(ids.long(), w)
    return _embedding_fwd(ids.long(), w)
