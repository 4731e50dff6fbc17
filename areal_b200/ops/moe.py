"""Mixture-of-experts routing and expert MLPs.

``moe_experts_forward`` computes ``sum_j w[t,j] * MLP_{idx[t,j]}(x[t])`` with SwiGLU
experts. On a B200 everything runs in this library's kernels and stays on the device:

* ``route``            softmax + top-k (+ renormalisation)              ``csrc/moe.cu``
* ``sort_by_expert``   stable counting sort of the ``[T*k]`` copies into a layout whose
                       per-expert segments are padded to 128 rows, plus the tile table
                       of the grouped GEMM (no host synchronisation)
* gather / combine     permutation into that layout and the weighted sum back
* grouped GEMMs        forward, dgrad and wgrad of all experts in one tcgen05 launch
                       each (``b200_gemm_grouped*`` in ``csrc/gemm_bf16.cu``)

The PyTorch restatement below (a loop over experts) is the CPU path and the oracle of
the GPU tests. Ordering semantics follow the reference's token reorderer
(areal/experimental/models/archon/moe/token_reorderer.py: copies sorted by expert,
ties by flat index) and its grouped experts (moe/grouped_experts.py).
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from . import _lib, fused
from .gemm import linear


# --------------------------------------------------------------------------- references


def route_ref(logits: torch.Tensor, k: int, renorm: bool):
    probs = logits.float().softmax(-1)
    w, idx = probs.topk(k, dim=-1)
    if renorm:
        w = w / w.sum(-1, keepdim=True)
    return idx.to(torch.int32), w


def permute_by_expert(idx: torch.Tensor, num_experts: int):
    """``idx [T, k]`` → (order [T*k]: flat copy indices sorted by expert, counts [E])."""
    flat = idx.reshape(-1).long()
    order = torch.argsort(flat, stable=True)
    counts = torch.bincount(flat, minlength=num_experts)
    return order, counts


def moe_experts_ref(x, idx, w, gate_up, down):
    T, H = x.shape
    k = idx.shape[1]
    E = gate_up.shape[0]
    order, counts = permute_by_expert(idx, E)
    token_of = order // k
    xs = x.index_select(0, token_of)
    offs = [0] + torch.cumsum(counts, 0).tolist()
    pieces = []
    for e in range(E):
        a, b = offs[e], offs[e + 1]
        if a == b:
            continue
        h = fused.swiglu(linear(xs[a:b], gate_up[e]))
        pieces.append(linear(h, down[e]))
    outs = torch.cat(pieces, 0) if pieces else torch.zeros((0, H), dtype=x.dtype, device=x.device)
    wflat = w.reshape(-1).index_select(0, order).to(outs.dtype)
    out = torch.zeros((T, H), dtype=torch.float32, device=x.device)
    out.index_add_(0, token_of, (outs * wflat[:, None]).float())
    return out.to(x.dtype)


# --------------------------------------------------------------------------- CUDA pieces


def route(logits: torch.Tensor, k: int, renorm: bool):
    """``logits [T, E]`` fp32 → ``(idx [T,k] int32, w [T,k] fp32)``."""
    T, E = logits.shape
    if not (_lib.use_cuda_kernels(logits) and logits.dtype == torch.float32 and E <= 256 and k <= 32):
        return route_ref(logits, k, renorm)
    logits = logits if logits.is_contiguous() else logits.contiguous()
    idx = torch.empty((T, k), dtype=torch.int32, device=logits.device)
    w = torch.empty((T, k), dtype=torch.float32, device=logits.device)
    rc = _lib.kernels().b200_moe_route(_lib.ptr(logits), _lib.ptr(idx), _lib.ptr(w), ctypes.c_int(T), ctypes.c_int(E),
                                       ctypes.c_int(k), ctypes.c_int(int(renorm)), _lib.stream_ptr())
    _lib.check(rc, "b200_moe_route")
    _lib.count_launch()
    return idx, w


@dataclass
class ExpertSort:
    """Device-side result of the sort; nothing here has been read back by the host."""

    n: int                     # T * k
    k: int
    num_experts: int
    max_rows: int              # rows allocated for padded buffers (multiple of 128)
    dest: torch.Tensor         # [n] padded row of every (token, choice) copy
    src_of: torch.Tensor       # [max_rows] flat copy index of every padded row, -1 for padding
    counts: torch.Tensor       # [E]
    prow0: torch.Tensor        # [E + 1] first padded row of every expert
    tile_expert: torch.Tensor  # [max_rows / 128] expert of every 128-row tile
    num_vm: torch.Tensor       # [1] number of tiles in use


def sort_by_expert(idx: torch.Tensor, num_experts: int) -> ExpertSort:
    T, k = idx.shape
    n = T * k
    dev = idx.device
    max_vm = (n + 127) // 128 + num_experts
    idx = idx.to(torch.int32).contiguous()
    ints = lambda m: torch.empty(m, dtype=torch.int32, device=dev)
    s = ExpertSort(n, k, num_experts, max_vm * 128, ints(n), ints(max_vm * 128), ints(num_experts),
                   ints(num_experts + 1), ints(max_vm), ints(1))
    chunk_hist = ints(max((n + 255) // 256, 1) * num_experts)
    if _lib.checked():
        _lib.check_index("moe_sort.expert_ids", idx, num_experts)
    rc = _lib.kernels().b200_moe_sort(_lib.ptr(idx), ctypes.c_int(n), ctypes.c_int(num_experts), _lib.ptr(chunk_hist),
                                      _lib.ptr(s.counts), _lib.ptr(s.prow0), _lib.ptr(s.tile_expert),
                                      _lib.ptr(s.num_vm), _lib.ptr(s.dest), _lib.ptr(s.src_of), ctypes.c_int(max_vm),
                                      _lib.stream_ptr())
    _lib.check(rc, "b200_moe_sort")
    _lib.count_launch(4)
    return s


def gather_rows(x: torch.Tensor, s: ExpertSort, scale: torch.Tensor | None = None) -> torch.Tensor:
    """``out[r] = scale[c] * x[c // k]`` for the copy ``c`` that lives in padded row ``r`` (zeros for padding)."""
    H = x.shape[1]
    out = torch.empty((s.max_rows, H), dtype=x.dtype, device=x.device)
    x = x if x.stride(1) == 1 else x.contiguous()
    rc = _lib.kernels().b200_moe_gather(_lib.ptr(x), ctypes.c_longlong(x.stride(0)), _lib.ptr(s.src_of),
                                        _lib.ptr(scale), _lib.ptr(s.num_vm), ctypes.c_int(s.k), ctypes.c_int(H),
                                        _lib.ptr(out), ctypes.c_int(s.max_rows), _lib.stream_ptr())
    _lib.check(rc, "b200_moe_gather")
    _lib.count_launch()
    return out


def combine_rows(y: torch.Tensor, s: ExpertSort, w: torch.Tensor | None) -> torch.Tensor:
    """``out[t] = sum_j w[t,j] * y[dest[t,j]]`` (plain sum when ``w`` is None)."""
    H = y.shape[1]
    T = s.n // s.k
    out = torch.empty((T, H), dtype=y.dtype, device=y.device)
    rc = _lib.kernels().b200_moe_combine(_lib.ptr(y), _lib.ptr(s.dest), _lib.ptr(w), ctypes.c_int(T), ctypes.c_int(s.k),
                                         ctypes.c_int(H), _lib.ptr(out), _lib.stream_ptr())
    _lib.check(rc, "b200_moe_combine")
    _lib.count_launch()
    return out


def grouped_gemm(a: torch.Tensor, w: torch.Tensor, s: ExpertSort, transpose_w: bool = True) -> torch.Tensor:
    """Per-expert product over padded rows. ``transpose_w``: ``a[r] @ w[e].T`` with ``w [E, N, K]``
    (forward); otherwise ``a[r] @ w[e]`` with ``w [E, K, N]`` (dgrad)."""
    E = w.shape[0]
    K = a.shape[1]
    N = w.shape[1] if transpose_w else w.shape[2]
    assert w.is_contiguous() and a.is_contiguous() and (w.shape[2] if transpose_w else w.shape[1]) == K
    out = torch.empty((s.max_rows, N), dtype=a.dtype, device=a.device)
    rc = _lib.kernels().b200_gemm_grouped(_lib.ptr(a), _lib.ptr(w), _lib.ptr(out), _lib.ptr(s.tile_expert),
                                          _lib.ptr(s.num_vm), ctypes.c_int(s.max_rows), ctypes.c_int(E),
                                          ctypes.c_int(N), ctypes.c_int(K), ctypes.c_int(0 if transpose_w else 1),
                                          _lib.stream_ptr())
    _lib.check(rc, "b200_gemm_grouped")
    _lib.count_launch()
    return out


def grouped_wgrad(dy: torch.Tensor, x: torch.Tensor, s: ExpertSort, out: torch.Tensor | None = None,
                  accumulate: bool = False, dtype=torch.bfloat16) -> torch.Tensor:
    """``dW[e] (+)= dy_e.T @ x_e`` → ``[E, N, K]``; ``out`` may be an fp32 main-grad buffer."""
    E, N, K = s.num_experts, dy.shape[1], x.shape[1]
    if out is None:
        out = torch.empty((E, N, K), dtype=dtype, device=dy.device)
    rc = _lib.kernels().b200_gemm_grouped_wgrad(_lib.ptr(dy), _lib.ptr(x), _lib.ptr(out), _lib.ptr(s.prow0),
                                                ctypes.c_int(s.max_rows), ctypes.c_int(E), ctypes.c_int(N),
                                                ctypes.c_int(K), ctypes.c_int(int(out.dtype == torch.float32)),
                                                ctypes.c_int(int(accumulate)), _lib.stream_ptr())
    _lib.check(rc, "b200_gemm_grouped_wgrad")
    _lib.count_launch()
    return out


def _swiglu_raw(gu: torch.Tensor) -> torch.Tensor:
    inter = gu.shape[1] // 2
    out = torch.empty((gu.shape[0], inter), dtype=gu.dtype, device=gu.device)
    rc = _lib.kernels().b200_swiglu_fwd(_lib.ptr(gu), _lib.ptr(out), ctypes.c_longlong(gu.shape[0]), ctypes.c_int(inter),
                                        _lib.stream_ptr())
    _lib.check(rc, "b200_swiglu_fwd")
    _lib.count_launch()
    return out


def _swiglu_bwd_raw(dy: torch.Tensor, gu: torch.Tensor) -> torch.Tensor:
    dgu = torch.empty_like(gu)
    rc = _lib.kernels().b200_swiglu_bwd(_lib.ptr(dy), _lib.ptr(gu), _lib.ptr(dgu), ctypes.c_longlong(gu.shape[0]),
                                        ctypes.c_int(gu.shape[1] // 2), _lib.stream_ptr())
    _lib.check(rc, "b200_swiglu_bwd")
    _lib.count_launch()
    return dgu


class _MoEExperts(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, idx, w, gate_up, down):
        E = gate_up.shape[0]
        s = sort_by_expert(idx, E)
        w32 = w.float().contiguous()
        xs = gather_rows(x, s)
        h1 = grouped_gemm(xs, gate_up, s)
        a = _swiglu_raw(h1)
        y = grouped_gemm(a, down, s)
        out = combine_rows(y, s, w32)
        ctx.save_for_backward(xs, h1, y, w32, gate_up, down)
        ctx.sort = s
        ctx.w_dtype = w.dtype
        return out

    @staticmethod
    def backward(ctx, dout):
        xs, h1, y, w32, gate_up, down = ctx.saved_tensors
        s: ExpertSort = ctx.sort
        dout = dout.contiguous()
        H = dout.shape[1]
        lib = _lib.kernels()
        dw = torch.empty((s.n,), dtype=torch.float32, device=dout.device)
        rc = lib.b200_moe_combine_dw(_lib.ptr(dout), _lib.ptr(y), _lib.ptr(s.dest), ctypes.c_int(s.n), ctypes.c_int(s.k),
                                     ctypes.c_int(H), _lib.ptr(dw), _lib.stream_ptr())
        _lib.check(rc, "b200_moe_combine_dw")
        _lib.count_launch()
        dy = gather_rows(dout, s, scale=w32.reshape(-1))
        a = _swiglu_raw(h1)
        da = grouped_gemm(dy, down, s, transpose_w=False)
        d_down = _wgrad_into(down, dy, a, s)
        dh1 = _swiglu_bwd_raw(da, h1)
        d_gate_up = _wgrad_into(gate_up, dh1, xs, s)
        dxs = grouped_gemm(dh1, gate_up, s, transpose_w=False)
        dx = combine_rows(dxs, s, None)
        return dx, None, dw.view(-1, s.k).to(ctx.w_dtype), d_gate_up, d_down


def _wgrad_into(param, dy, x, s):
    """Expert weight gradient; accumulates straight into ``param.main_grad`` (fp32) when the engine set one."""
    main = getattr(param, "main_grad", None)
    if main is not None:
        grouped_wgrad(dy, x, s, out=main, accumulate=True)
        return None
    return grouped_wgrad(dy, x, s, dtype=param.dtype)


def moe_experts_forward(x, idx, w, gate_up, down):
    """``x [T,H]``, ``idx [T,k]``, ``w [T,k]``, ``gate_up [E,2I,H]``, ``down [E,H,I]`` → ``[T,H]``."""
    E, I2, H = gate_up.shape
    ok = (_lib.use_cuda_kernels(x, gate_up, down) and x.dtype == torch.bfloat16 and H % 128 == 0 and I2 % 128 == 0
          and (I2 // 2) % 64 == 0 and E <= 1024)
    if not ok:
        return moe_experts_ref(x, idx, w, gate_up, down)
    return _MoEExperts.apply(x.contiguous(), idx, w, gate_up, down)
