"""Block-scaled fp8 (e4m3): quantisation, dequantisation, GEMM and an fp8 linear.

Recipe: activations are quantised per 1x128 group, weights per 128x128 block
(bf16 master weights stay authoritative), products accumulate in fp32 with a
promotion every 128-wide K block (``csrc/quant_fp8.cu``, ``csrc/gemm_fp8_block.cu``).
``ue8m0=True`` rounds scales up to powers of two (the Blackwell scale format).
The forward GEMM of :func:`fp8_linear` runs in fp8; both backward GEMMs run on
the bf16 tcgen05 kernel against the bf16 master weight.

Reference: areal/engine/megatron_utils/fp8/{kernels,quantize,ue8m0}.py and
areal/experimental/models/archon/fp8.py:134-230.
"""

from __future__ import annotations

import ctypes

import torch

from . import _lib
from .gemm import gemm

FP8_MAX = 448.0
FP8 = torch.float8_e4m3fn


def _round_pow2(s: torch.Tensor) -> torch.Tensor:
    return torch.exp2(torch.ceil(torch.log2(s)))


def quant_block128_ref(x: torch.Tensor, ue8m0: bool = False):
    M, N = x.shape
    mb, nb = -(-M // 128), -(-N // 128)
    xp = torch.zeros(mb * 128, nb * 128, dtype=torch.float32, device=x.device)
    xp[:M, :N] = x.float()
    blocks = xp.view(mb, 128, nb, 128)
    amax = blocks.abs().amax(dim=(1, 3)).clamp(min=1e-12)
    scale = amax / FP8_MAX
    if ue8m0:
        scale = _round_pow2(scale)
    q = (blocks / scale[:, None, :, None]).clamp(-FP8_MAX, FP8_MAX).view(mb * 128, nb * 128)[:M, :N]
    return q.to(FP8), scale


def quant_1x128_ref(x: torch.Tensor, ue8m0: bool = False):
    M, K = x.shape
    g = -(-K // 128)
    xp = torch.zeros(M, g * 128, dtype=torch.float32, device=x.device)
    xp[:, :K] = x.float()
    groups = xp.view(M, g, 128)
    scale = groups.abs().amax(-1).clamp(min=1e-12) / FP8_MAX
    if ue8m0:
        scale = _round_pow2(scale)
    q = (groups / scale[..., None]).clamp(-FP8_MAX, FP8_MAX).view(M, g * 128)[:, :K]
    return q.to(FP8), scale


def dequant_ref(q: torch.Tensor, scale: torch.Tensor, block_m: int) -> torch.Tensor:
    M, N = q.shape
    s = scale.repeat_interleave(128, 1)[:, :N]
    if block_m != 1:
        s = s.repeat_interleave(128, 0)[:M]
    return (q.float() * s).to(torch.bfloat16)


def quant_fp8_block128(x: torch.Tensor, ue8m0: bool = False):
    """Weights: ``x [M,N]`` bf16 → ``(fp8 [M,N], scale [ceil(M/128), ceil(N/128)] fp32)``."""
    if not _lib.use_cuda_kernels(x):
        return quant_block128_ref(x, ue8m0)
    x = x if x.stride(1) == 1 else x.contiguous()
    M, N = x.shape
    y = torch.empty((M, N), dtype=FP8, device=x.device)
    scale = torch.empty((-(-M // 128), -(-N // 128)), dtype=torch.float32, device=x.device)
    rc = _lib.kernels().b200_quant_fp8_block128(_lib.ptr(x), ctypes.c_longlong(x.stride(0)), _lib.ptr(y),
                                                ctypes.c_longlong(y.stride(0)), _lib.ptr(scale), ctypes.c_int(M),
                                                ctypes.c_int(N), ctypes.c_int(int(ue8m0)), _lib.stream_ptr())
    _lib.check(rc, "b200_quant_fp8_block128")
    _lib.count_launch()
    return y, scale


def quant_fp8_1x128(x: torch.Tensor, ue8m0: bool = False):
    """Activations: ``x [M,K]`` bf16 → ``(fp8 [M,K], scale [M, ceil(K/128)] fp32)``."""
    if not _lib.use_cuda_kernels(x):
        return quant_1x128_ref(x, ue8m0)
    x = x if x.stride(1) == 1 else x.contiguous()
    M, K = x.shape
    y = torch.empty((M, K), dtype=FP8, device=x.device)
    scale = torch.empty((M, -(-K // 128)), dtype=torch.float32, device=x.device)
    rc = _lib.kernels().b200_quant_fp8_1x128(_lib.ptr(x), ctypes.c_longlong(x.stride(0)), _lib.ptr(y),
                                             ctypes.c_longlong(y.stride(0)), _lib.ptr(scale),
                                             ctypes.c_longlong(scale.stride(0)), ctypes.c_int(M), ctypes.c_int(K),
                                             ctypes.c_int(int(ue8m0)), _lib.stream_ptr())
    _lib.check(rc, "b200_quant_fp8_1x128")
    _lib.count_launch()
    return y, scale


def dequant_fp8(q: torch.Tensor, scale: torch.Tensor, block_m: int = 128) -> torch.Tensor:
    if not _lib.use_cuda_kernels(q):
        return dequant_ref(q, scale, block_m)
    M, N = q.shape
    y = torch.empty((M, N), dtype=torch.bfloat16, device=q.device)
    rc = _lib.kernels().b200_dequant_fp8(_lib.ptr(q), ctypes.c_longlong(q.stride(0)), _lib.ptr(scale),
                                         ctypes.c_longlong(scale.stride(0)), _lib.ptr(y),
                                         ctypes.c_longlong(y.stride(0)), ctypes.c_int(M), ctypes.c_int(N),
                                         ctypes.c_int(block_m), _lib.stream_ptr())
    _lib.check(rc, "b200_dequant_fp8")
    _lib.count_launch()
    return y


def gemm_fp8_block_ref(a8, sa, b8, sb):
    a = dequant_ref(a8, sa, 1).float()
    b = dequant_ref(b8, sb, 128).float()
    return (a @ b.t()).to(torch.bfloat16)


def gemm_fp8_block(a8, sa, b8, sb) -> torch.Tensor:
    """``C[M,N] = dequant(a8, sa) @ dequant(b8, sb).T`` computed in fp8 with per-K-block promotion."""
    if not _lib.use_cuda_kernels(a8, b8):
        return gemm_fp8_block_ref(a8, sa, b8, sb)
    M, K = a8.shape
    N = b8.shape[0]
    assert K % 16 == 0 and a8.stride(1) == 1 and b8.stride(1) == 1
    c = torch.empty((M, N), dtype=torch.bfloat16, device=a8.device)
    rc = _lib.kernels().b200_gemm_fp8_block(_lib.ptr(a8), _lib.ptr(b8), _lib.ptr(sa),
                                            ctypes.c_longlong(sa.stride(0)), _lib.ptr(sb),
                                            ctypes.c_longlong(sb.stride(0)), _lib.ptr(c), ctypes.c_int(M),
                                            ctypes.c_int(N), ctypes.c_int(K), ctypes.c_longlong(a8.stride(0)),
                                            ctypes.c_longlong(b8.stride(0)), ctypes.c_longlong(c.stride(0)),
                                            _lib.stream_ptr())
    _lib.check(rc, "b200_gemm_fp8_block")
    _lib.count_launch()
    return c


class _FP8Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, ue8m0):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        a8, sa = quant_fp8_1x128(x2, ue8m0)
        cache = getattr(w, "_fp8_cache", None)
        if cache is None or cache[0] != w._version:
            b8, sb = quant_fp8_block128(w.detach(), ue8m0)
            try:
                w._fp8_cache = (w._version, b8, sb)
            except AttributeError:
                pass
        else:
            _, b8, sb = cache
        y = gemm_fp8_block(a8, sa, b8, sb)
        ctx.save_for_backward(x2, w)
        ctx.in_shape = shape
        return y.reshape(*shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1]).to(x2.dtype)
        dx = gemm(dy2, w, b_mn=True, out_dtype=x2.dtype).reshape(ctx.in_shape) if ctx.needs_input_grad[0] else None
        dw = None
        if ctx.needs_input_grad[1]:
            main = getattr(w, "main_grad", None)
            if main is not None:
                gemm(dy2, x2, a_mn=True, b_mn=True, out=main, accumulate=True)
            else:
                dw = gemm(dy2, x2, a_mn=True, b_mn=True, out_dtype=w.dtype)
        return dx, dw, None


def fp8_linear(x: torch.Tensor, w: torch.Tensor, ue8m0: bool = True) -> torch.Tensor:
    """``x @ w.T`` with the forward product in block-scaled fp8 (bf16 master weight ``w``)."""
    if x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 16 == 0:
        return _FP8Linear.apply(x, w, ue8m0)
    a8, sa = quant_1x128_ref(x.reshape(-1, x.shape[-1]), ue8m0)
    b8, sb = quant_block128_ref(w, ue8m0)
    y = dequant_ref(a8, sa, 1).float() @ dequant_ref(b8, sb, 128).float().t()
    return y.to(x.dtype).reshape(*x.shape[:-1], w.shape[0])
