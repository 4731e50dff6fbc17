"""Mixture-of-experts token routing and expert MLPs.

``moe_experts_forward`` computes ``sum_k w[t,k] * MLP_{idx[t,k]}(x[t])`` with
SwiGLU experts. Tokens are grouped by expert (stable sort of the flattened
``[T*k]`` assignments, as the reference's token reorderer does,
areal/experimental/models/archon/moe/token_reorderer.py), each expert's slice
goes through the GEMM kernel, and the weighted results are scattered back
(areal/experimental/models/archon/moe/moe.py).
"""

from __future__ import annotations

import torch

from . import fused
from .gemm import linear


def permute_by_expert(idx: torch.Tensor, num_experts: int):
    """``idx [T, k]`` → (order [T*k] token-copy indices sorted by expert,
    counts [E], token_of_copy [T*k])."""
    flat = idx.reshape(-1)
    order = torch.argsort(flat, stable=True)
    counts = torch.bincount(flat, minlength=num_experts)
    return order, counts


def moe_experts_forward(x, idx, w, gate_up, down):
    T, H = x.shape
    k = idx.shape[1]
    E = gate_up.shape[0]
    order, counts = permute_by_expert(idx, E)
    token_of = order // k
    xs = x.index_select(0, token_of)  # [T*k, H] grouped by expert
    outs = torch.empty((T * k, H), dtype=x.dtype, device=x.device)
    offs = [0] + torch.cumsum(counts, 0).tolist()
    pieces = []
    for e in range(E):
        a, b = offs[e], offs[e + 1]
        if a == b:
            continue
        h = fused.swiglu(linear(xs[a:b], gate_up[e]))
        pieces.append((a, b, linear(h, down[e])))
    if pieces:
        outs = torch.cat([p[2] for p in pieces], 0)
    wflat = w.reshape(-1).index_select(0, order).to(outs.dtype)
    out = torch.zeros((T, H), dtype=torch.float32, device=x.device)
    out.index_add_(0, token_of, (outs * wflat[:, None]).float())
    return out.to(x.dtype)
