"""bf16 GEMM on the tcgen05 kernel (``csrc/gemm_bf16.cu``) and the autograd
``linear`` built on it.

The three products of a linear layer run on one kernel by choosing operand
majors instead of materialising transposes:

* forward  ``y  = x W^T``  – both operands K-major
* dgrad    ``dx = dy W``   – ``W`` read MN-major
* wgrad    ``dW = dy^T x`` – both operands MN-major, fp32 output with optional
  accumulation into a main-grad buffer.

Counterpart of the cuBLAS-backed ``nn.Linear`` calls of the reference
(areal/experimental/models/archon/qwen3/model/model.py:103-293).
"""

from __future__ import annotations

import ctypes

import torch

from . import _lib, wgrad_defer


def _gemm_ref(a, b, a_mn, b_mn, bias, out_dtype, out, accumulate):
    A = a.t() if a_mn else a
    B = b.t() if b_mn else b
    c = A.float() @ B.float().t()
    if bias is not None:
        c = c + bias.float()
    if out is not None:
        if accumulate:
            out.add_(c.to(out.dtype))
        else:
            out.copy_(c.to(out.dtype))
        return out
    return c.to(out_dtype)


def gemm(
    a: torch.Tensor,
    b: torch.Tensor,
    *,
    a_mn: bool = False,
    b_mn: bool = False,
    bias: torch.Tensor | None = None,
    out: torch.Tensor | None = None,
    out_dtype: torch.dtype = torch.bfloat16,
    accumulate: bool = False,
    bn: int = 0,
) -> torch.Tensor:
    """``C[M,N] = A B^T (+bias)``.

    ``a`` is ``[M,K]`` (``a_mn=False``) or ``[K,M]`` (``a_mn=True``); ``b`` is ``[N,K]``
    or ``[K,N]`` likewise. ``out`` may be a bf16 or fp32 2-D tensor with unit
    inner stride; ``accumulate`` adds to it.
    """
    if not _lib.use_cuda_kernels(a, b):
        return _gemm_ref(a, b, a_mn, b_mn, bias, out_dtype, out, accumulate)
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16, "bf16 operands required"
    assert a.dim() == 2 and b.dim() == 2
    if a.stride(1) != 1 or (a.stride(0) % 8) or (a.data_ptr() % 16):
        a = a.contiguous()
    if b.stride(1) != 1 or (b.stride(0) % 8) or (b.data_ptr() % 16):
        b = b.contiguous()
    if a_mn:
        K, M = a.shape
    else:
        M, K = a.shape
    if b_mn:
        Kb, N = b.shape
    else:
        N, Kb = b.shape
    assert K == Kb, f"reduction dims differ: {K} vs {Kb}"
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
        accumulate = False
    assert out.shape == (M, N) and out.stride(1) == 1
    assert out.dtype in (torch.bfloat16, torch.float32)
    # TMA needs 16-byte aligned pitches: pad the contiguous extent when it is not.
    need_pad = (a.shape[1] % 8) or (b.shape[1] % 8)
    if need_pad:
        def pad(t):
            p = (-t.shape[1]) % 8
            return torch.nn.functional.pad(t, (0, p)) if p else t
        a, b = pad(a), pad(b)
        if not a_mn:
            K = a.shape[1]
    # skinny products (decode steps): too few output tiles for 148 SMs ⇒ split the K extent
    if (bn == 0 and not a_mn and not b_mn and not accumulate and out.dtype == torch.bfloat16 and M <= 512
            and N % 4 == 0 and out.stride(0) % 4 == 0 and not need_pad and K >= 1024):
        tiles = -(-M // 128) * -(-N // 128)
        splits = min(8, 148 // tiles, K // 256)
        if splits >= 2:
            ws = torch.empty((splits * -(-M // 128) * 128, N), dtype=torch.float32, device=a.device)
            rc = _lib.kernels().b200_gemm_bf16_splitk(
                _lib.ptr(a), _lib.ptr(b), _lib.ptr(out), _lib.ptr(bias), _lib.ptr(ws), ctypes.c_int(M), ctypes.c_int(N),
                ctypes.c_int(K), ctypes.c_longlong(a.stride(0)), ctypes.c_longlong(b.stride(0)),
                ctypes.c_longlong(out.stride(0)), ctypes.c_int(splits), _lib.stream_ptr())
            _lib.check(rc, "b200_gemm_bf16_splitk")
            _lib.count_launch(2)
            return out
    if bn == 0:
        bn = 256 if N > 128 else 128
        if bn == 256:
            # Prefer 128-wide tiles when 256-wide ones would leave most SMs idle.
            tiles256 = -(-M // 128) * -(-N // 256)
            if tiles256 < 100:
                bn = 128
    lib = _lib.kernels()
    fn = lib.b200_gemm_bf16
    fn.restype = ctypes.c_int
    rc = fn(
        _lib.ptr(a), _lib.ptr(b), _lib.ptr(out), _lib.ptr(bias),
        ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(K),
        ctypes.c_longlong(a.stride(0)), ctypes.c_longlong(b.stride(0)),
        ctypes.c_longlong(out.stride(0)),
        ctypes.c_int(int(a_mn)), ctypes.c_int(int(b_mn)),
        ctypes.c_int(int(out.dtype == torch.float32)), ctypes.c_int(int(accumulate)),
        ctypes.c_int(bn), _lib.stream_ptr(),
    )
    _lib.check(rc, "b200_gemm_bf16")
    _lib.count_launch()
    return out


def _splitk_plan(M: int, N: int, K: int) -> int:
    """Number of K splits the skinny-GEMM path uses for this shape (0: not a split-K shape)."""
    if M > 512 or N % 4 or K < 1024:
        return 0
    tiles = -(-M // 128) * -(-N // 128)
    splits = min(8, 148 // tiles, K // 256)
    return splits if splits >= 2 else 0


@torch.no_grad()
def linear_rmsnorm(x: torch.Tensor, w: torch.Tensor, norm_w: torch.Tensor, eps: float,
                   residual: torch.Tensor | None = None):
    """``h = x @ w.T (+ residual)``; returns ``(rmsnorm(h) * norm_w, h)``: a decoder block's projection,
    residual add and following norm. For skinny (decode-step) shapes the residual add and the norm
    run inside the split-K reduction kernel (two launches instead of three, bit-identical results);
    other shapes run the separate kernels. Inference only."""
    from . import fused

    M, K = x.shape
    N = w.shape[0]
    splits = _splitk_plan(M, N, K) if (_lib.use_cuda_kernels(x, w) and x.dtype == torch.bfloat16) else 0
    ok = (splits and N % 8 == 0 and N <= 8192 and K % 8 == 0 and x.stride(1) == 1 and w.stride(1) == 1
          and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
          and (residual is None or residual.is_contiguous()) and norm_w.is_contiguous())
    if not ok:
        a = linear(x, w)
        if residual is None:
            return fused.rmsnorm(a, norm_w, eps), a
        return fused.rmsnorm(a, norm_w, eps, residual=residual)
    ws = torch.empty((splits * -(-M // 128) * 128, N), dtype=torch.float32, device=x.device)
    y = torch.empty((M, N), dtype=x.dtype, device=x.device)
    res_out = torch.empty((M, N), dtype=x.dtype, device=x.device)
    rc = _lib.kernels().b200_gemm_bf16_splitk_rmsnorm(
        _lib.ptr(x), _lib.ptr(w), None, _lib.ptr(ws), ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(K),
        ctypes.c_longlong(x.stride(0)), ctypes.c_longlong(w.stride(0)), ctypes.c_int(splits), _lib.ptr(residual),
        _lib.ptr(norm_w), _lib.ptr(y), _lib.ptr(res_out), ctypes.c_float(eps), _lib.stream_ptr())
    _lib.check(rc, "b200_gemm_bf16_splitk_rmsnorm")
    _lib.count_launch(2)
    return y, res_out


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        y = gemm(x2, w, bias=bias, out_dtype=x.dtype)
        ctx.save_for_backward(x2, w)
        ctx.has_bias = bias is not None
        ctx.in_shape = shape
        return y.reshape(*shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if dy2.dtype != x2.dtype:
            dy2 = dy2.to(x2.dtype)
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, w, b_mn=True, out_dtype=x2.dtype).reshape(ctx.in_shape)
        if ctx.needs_input_grad[1]:
            main = getattr(w, "main_grad", None)
            queue = wgrad_defer.active()
            if queue is not None and (main is not None or w.is_leaf):
                # zero-bubble pipeline schedules: the weight-gradient GEMM is parked and runs in a later W action
                if main is not None:
                    queue.push(lambda: gemm(dy2, x2, a_mn=True, b_mn=True, out=main, accumulate=True))
                else:
                    queue.push(lambda: wgrad_defer.accumulate(
                        w, gemm(dy2, x2, a_mn=True, b_mn=True, out_dtype=w.dtype)))
            elif main is not None:
                # fp32 main-grad accumulation across micro-batches, fused in the epilogue
                gemm(dy2, x2, a_mn=True, b_mn=True, out=main, accumulate=True)
                dw = None
            else:
                dw = gemm(dy2, x2, a_mn=True, b_mn=True, out_dtype=w.dtype)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.float().sum(0).to(dy2.dtype)
        return dx, dw, db


def linear(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """``x @ w.T + bias`` with forward and both backward products on the tcgen05 kernel."""
    if x.is_cuda and x.dtype == torch.bfloat16:
        return _Linear.apply(x, w, bias)
    if wgrad_defer.armed() and torch.is_grad_enabled():
        return wgrad_defer.SplitLinear.apply(x, w, bias)
    return torch.nn.functional.linear(x, w, bias)
