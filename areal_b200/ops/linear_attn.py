"""Linear-attention ops for hybrid models on packed sequences (``csrc/linear_attn.cu``):
causal depthwise conv1d (+SiLU) with forward and backward kernels, and the gated delta rule /
simple gated linear attention recurrences. The recurrences run their CUDA kernel whenever no
gradient is needed (rollout, logprob recomputation); under autograd they run the chunk-parallel
PyTorch form below (``linear_attn_chunked``: one sequential step per 64 tokens). The per-token
restatement (``linear_attn_ref``) is the test oracle of both.

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


def linear_attn_chunked(q, k, v, a, b, cu, scale: float, mode: str, chunk: int = 64, return_state: bool = False):
    """The same recurrences in chunk-parallel form (differentiable; the training path).

    Inside a chunk that starts from state ``S0``, with ``G_i`` the running sum of ``log a`` and
    ``D_ij = exp(G_i - G_j)`` for ``j <= i``:

    * the delta-rule writes ``u_i = b_i (v_i - (a_i S_{i-1})^T k_i)`` solve the unit lower-triangular
      system ``(I + A) U = diag(b) (V - diag(exp G) K S0)`` with ``A_ij = b_i D_ij (k_i . k_j)``, ``j < i``
      (``U = V`` for ``simple_gla``);
    * ``O = scale * (diag(exp G) Q S0 + (D o Q K^T) U)`` and ``S_C = exp(G_C) S0 + (K o exp(G_C - G))^T U``.

    ``(I + A)^-1`` does not depend on the state, so it is computed for all chunks of a sequence at
    once; only the small ``S0`` recursion is sequential (one step per chunk, not per token)."""
    T, H, DK = q.shape
    DV = v.shape[2]
    delta = mode == "gated_delta"
    outs = []
    finals = []  # per sequence: the state after its last token (``return_state``)
    cu_l = [int(c) for c in cu]
    for s0, s1 in zip(cu_l[:-1], cu_l[1:]):
        L = s1 - s0
        if L == 0:
            finals.append(torch.zeros(H, DK, DV, dtype=torch.float32, device=q.device))
            continue
        n = -(-L // chunk)
        pad = n * chunk - L

        def prep(t, fill=0.0):  # [L, H, ...] -> [H, n, chunk, ...]
            t = t[s0:s1].float()
            if pad:
                t = torch.cat([t, t.new_full((pad,) + tuple(t.shape[1:]), fill)], 0)
            return t.reshape(n, chunk, *t.shape[1:]).movedim(2, 0)

        Q, K, V = prep(q), prep(k), prep(v)
        G = prep(a, 1.0).clamp_min(1e-30).log().cumsum(-1)             # [H, n, C]
        Dm = (G[..., :, None] - G[..., None, :]).tril().exp().tril()   # D_ij, j <= i
        eg = G.exp()[..., None]
        if delta:
            Bt = prep(b)[..., None]                                     # [H, n, C, 1]
            A = (Bt * Dm * (K @ K.transpose(-1, -2))).tril(-1)
            eye = torch.eye(chunk, device=q.device, dtype=torch.float32)
            rhs = torch.cat([Bt * V, Bt * eg * K], -1)                  # one solve for W_v and W_k
            sol = torch.linalg.solve_triangular(A + eye, rhs, upper=False, unitriangular=True)
            Wv, Wk = sol[..., :DV], sol[..., DV:]
        QK = Dm * (Q @ K.transpose(-1, -2))
        Kd = K * (G[..., -1:, None] - G[..., None]).exp()               # k_j exp(G_C - G_j)
        S = torch.zeros(H, DK, DV, dtype=torch.float32, device=q.device)
        o_chunks = []
        for c in range(n):
            U = (Wv[:, c] - Wk[:, c] @ S) if delta else V[:, c]
            o_chunks.append((eg[:, c] * Q[:, c]) @ S + QK[:, c] @ U)
            S = eg[:, c, -1][..., None] * S + Kd[:, c].transpose(-1, -2) @ U
        o = torch.stack(o_chunks, 1).reshape(H, n * chunk, DV)[:, :L]
        outs.append(o.transpose(0, 1))
        finals.append(S)  # padding rows have a = 1, k = v = 0: they leave the state untouched
    out = (torch.cat(outs, 0) * scale).to(q.dtype) if outs else torch.zeros_like(v)
    if return_state:
        return out, (torch.stack(finals) if finals else torch.zeros(0, H, DK, DV, device=q.device))
    return out


def linear_attn(q, k, v, a, b, cu, scale: float | None = None, mode: str = "gated_delta"):
    """``o_t = scale * S_t^T q_t`` with ``S_t = a_t S_{t-1} + k_t v_t^T`` (``simple_gla``) or the gated
    delta rule ``S_t = a_t S_{t-1} + b_t k_t (v_t - (a_t S_{t-1})^T k_t)^T``."""
    if mode not in ("gated_delta", "simple_gla"):
        raise ValueError(f"unknown linear-attention mode {mode!r}")
    T, H, DK = q.shape
    DV = v.shape[2]
    scale = scale if scale is not None else DK ** -0.5
    needs_grad = torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in (q, k, v, a, b))
    if needs_grad:
        return linear_attn_chunked(q, k, v, a, b, cu, scale, mode)
    if not (_lib.use_cuda_kernels(q, k, v) and q.dtype == torch.bfloat16 and DK in (64, 128) and DV <= 256):
        return linear_attn_chunked(q, k, v, a, b, cu, scale, mode) if T > 256 else \
            linear_attn_ref(q, k, v, a, b, cu, scale, mode)
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


@torch.no_grad()
def linear_attn_prefill(q, k, v, a, b, cu, scale: float | None = None, mode: str = "gated_delta"):
    """Inference prefill: outputs of every token AND the recurrent state after each sequence's last
    token (``[n_seq, H, DK, DV]`` fp32), which a decode step continues from."""
    T, H, DK = q.shape
    DV = v.shape[2]
    scale = scale if scale is not None else DK ** -0.5
    n_seq = int(cu.numel()) - 1
    if not (_lib.use_cuda_kernels(q, k, v) and q.dtype == torch.bfloat16 and DK in (64, 128) and DV <= 256):
        return linear_attn_chunked(q, k, v, a, b, cu, scale, mode, return_state=True)
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    a32 = a.float().contiguous()
    b32 = b.float().contiguous() if b is not None else None
    cu = cu.int().contiguous()
    o = torch.empty_like(v)
    state = torch.empty((n_seq, H, DK, DV), dtype=torch.float32, device=q.device)
    rc = _lib.kernels().b200_linear_attn_fwd(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(a32), _lib.ptr(b32),
                                             _lib.ptr(cu), _lib.ptr(o), _lib.ptr(state), ctypes.c_int(n_seq),
                                             ctypes.c_int(H), ctypes.c_int(DK), ctypes.c_int(DV), ctypes.c_float(scale),
                                             ctypes.c_int(1 if mode == "gated_delta" else 0), _lib.stream_ptr())
    _lib.check(rc, "b200_linear_attn_fwd")
    _lib.count_launch()
    return o, state


@torch.no_grad()
def linear_attn_step(q, k, v, a, b, state, scale: float | None = None, mode: str = "gated_delta"):
    """One decode step for a batch of sequences: ``q, k [B, H, DK]``, ``v [B, H, DV]``, ``a, b [B, H]``,
    ``state [B, H, DK, DV]`` fp32. Returns ``(o [B, H, DV], new_state)``; the same recurrence as
    :func:`linear_attn_ref` applied to one token (batched tensor ops: the state read / write dominates)."""
    DK = q.shape[-1]
    scale = scale if scale is not None else DK ** -0.5
    S = state * a.float()[..., None, None]
    kf, vf = k.float(), v.float()
    if mode == "gated_delta":
        u = torch.einsum("bhkv,bhk->bhv", S, kf)
        S = S + torch.einsum("bhk,bhv->bhkv", kf, b.float()[..., None] * (vf - u))
    else:
        S = S + torch.einsum("bhk,bhv->bhkv", kf, vf)
    o = torch.einsum("bhkv,bhk->bhv", S, q.float()) * scale
    return o.to(v.dtype), S
