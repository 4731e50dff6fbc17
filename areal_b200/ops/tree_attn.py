"""Tree (trie-packed) attention: sequences that share prefixes are merged into a trie and packed
in depth-first order, so every shared token is computed once. A key ``j`` is visible to a query
``i`` iff ``j`` is an ancestor of ``i`` (or ``i`` itself), which in depth-first order is the interval
test ``j <= i < exit[j]`` (``exit[j]`` = end of ``j``'s subtree). The tcgen05 attention kernels
take ``exit`` as an extra per-key array; everything else (tiles, GQA, backward) is the varlen path.

:func:`build_packed_tree` packs a list of token sequences; :func:`gather_sequences` maps per-node
outputs (logprobs, hidden states) back to the original sequences. Reference:
areal/models/tree_attn/{tree.py:41-366,triton_kernel.py,functional.py}.
"""

from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass

import numpy as np
import torch

from . import _lib
from .attention import _BT, _QT


@dataclass
class PackedTree:
    tokens: torch.Tensor        # [N] token ids in depth-first order (trees one after another)
    parent: torch.Tensor        # [N] parent node (-1 for roots)
    position_ids: torch.Tensor  # [N] depth of the node = position in its sequence
    exit: torch.Tensor          # [N] tree-relative end of the node's subtree
    tree_cu: list[int]          # boundaries of the trees inside the packed array
    seq_nodes: list[list[int]]  # for every input sequence the node index of each of its tokens

    @property
    def num_nodes(self) -> int:
        return int(self.tokens.numel())


def build_packed_tree(sequences: list[list[int]]) -> PackedTree:
    """Merges sequences by common prefix. Sequences with different first tokens form different
    trees; children are visited in first-seen order, so the packing is deterministic."""
    children: list[dict[int, int]] = []
    tok: list[int] = []
    par: list[int] = []
    roots: dict[int, int] = {}
    seq_path: list[list[int]] = []

    def new_node(t, p):
        tok.append(t)
        par.append(p)
        children.append({})
        return len(tok) - 1

    for s in sequences:
        path = []
        cur = -1
        for t in s:
            table = roots if cur < 0 else children[cur]
            nxt = table.get(t)
            if nxt is None:
                nxt = table[t] = new_node(t, cur)
            path.append(nxt)
            cur = nxt
        seq_path.append(path)
    # depth-first renumbering
    order: list[int] = []
    exit_of: dict[int, int] = {}
    depth: dict[int, int] = {}
    tree_cu = [0]
    for r in roots.values():
        base = len(order)
        stack = [(r, 0, False)]
        while stack:
            n, d, done = stack.pop()
            if done:
                exit_of[n] = len(order) - base
                continue
            depth[n] = d
            order.append(n)
            stack.append((n, d, True))
            for c in reversed(list(children[n].values())):
                stack.append((c, d + 1, False))
        tree_cu.append(len(order))
    new_id = {n: i for i, n in enumerate(order)}
    tokens = torch.tensor([tok[n] for n in order], dtype=torch.long)
    parent = torch.tensor([new_id[par[n]] if par[n] >= 0 else -1 for n in order], dtype=torch.long)
    pos = torch.tensor([depth[n] for n in order], dtype=torch.long)
    ex = torch.tensor([exit_of[n] for n in order], dtype=torch.int32)
    return PackedTree(tokens, parent, pos, ex, tree_cu, [[new_id[n] for n in p] for p in seq_path])


def gather_sequences(node_values: torch.Tensor, tree: PackedTree) -> list[torch.Tensor]:
    """Per-node values ``[N, ...]`` → one tensor per original sequence."""
    return [node_values[torch.tensor(p, dtype=torch.long, device=node_values.device)] for p in tree.seq_nodes]


class TreeMeta:
    """Tile tables of one packed-tree batch: every tree is one "sequence" of the varlen kernels."""

    def __init__(self, tree: PackedTree, device):
        cu = np.asarray(tree.tree_cu, dtype=np.int64)
        self.cu_cpu = cu
        self.total = int(cu[-1])
        ex = tree.exit.numpy()
        fwd, bwd = [], []
        for b in range(len(cu) - 1):
            s, e = int(cu[b]), int(cu[b + 1])
            L = e - s
            for q0 in range(0, L, _QT):
                fwd.append((s + q0, min(_QT, L - q0), s, min(L, q0 + _QT), q0, 0, 0, 0))
            for k0 in range(0, L, _BT):
                n = min(_BT, L - k0)
                # queries beyond the last subtree end of this key block see none of its keys
                reach = int(ex[s + k0:s + k0 + n].max())
                bwd.append((s + k0, n, k0, s, reach, 0, 0, 0))
        fwd.sort(key=lambda t: -t[3])
        bwd.sort(key=lambda t: -(t[4] - t[2]))
        self.n_fwd, self.n_bwd = len(fwd), len(bwd)
        self.fwd_tiles = torch.tensor(fwd, dtype=torch.int32).reshape(-1, 8).to(device)
        self.bwd_tiles = torch.tensor(bwd, dtype=torch.int32).reshape(-1, 8).to(device)
        self.key_exit = tree.exit.to(device=device, dtype=torch.int32).contiguous()


def ancestor_mask(tree: PackedTree) -> torch.Tensor:
    """Dense ``[N, N]`` boolean mask (query row, key column) from the parent pointers."""
    N = tree.num_nodes
    m = torch.zeros(N, N, dtype=torch.bool)
    for i in range(N):
        j = i
        while j >= 0:
            m[i, j] = True
            j = int(tree.parent[j])
    return m


def tree_attention_ref(q, k, v, tree: PackedTree, scale=None):
    T, Hq, D = q.shape
    g = Hq // k.shape[1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    mask = ancestor_mask(tree).to(q.device)
    qs = q.float().transpose(0, 1)
    ks = k.float().transpose(0, 1).repeat_interleave(g, 0)
    vs = v.float().transpose(0, 1).repeat_interleave(g, 0)
    att = (qs @ ks.transpose(1, 2) * scale).masked_fill(~mask, float("-inf")).softmax(-1)
    return (att @ vs).transpose(0, 1).to(q.dtype)


class _TreeAttn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, meta: TreeMeta, scale):
        T, Hq, D = q.shape
        Hkv = k.shape[1]
        q = q.contiguous()
        o = torch.empty_like(q)
        lse = torch.empty((Hq, T), dtype=torch.float32, device=q.device)
        rc = _lib.kernels().b200_attn_fwd_ex(
            _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(o), _lib.ptr(lse), _lib.ptr(meta.fwd_tiles),
            ctypes.c_int(meta.n_fwd), ctypes.c_int(T), ctypes.c_int(T), ctypes.c_int(Hq), ctypes.c_int(Hkv),
            ctypes.c_longlong(q.stride(0)), ctypes.c_longlong(k.stride(0)), ctypes.c_longlong(v.stride(0)),
            ctypes.c_float(scale), _lib.ptr(meta.key_exit), _lib.stream_ptr())
        _lib.check(rc, "b200_attn_fwd_ex")
        _lib.count_launch()
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.meta, ctx.scale = meta, scale
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse = ctx.saved_tensors
        meta = ctx.meta
        T, Hq, D = q.shape
        Hkv = k.shape[1]
        do = do.contiguous()
        dq_acc = torch.zeros((T, Hq, D), dtype=torch.float32, device=q.device)
        delta = torch.empty((Hq, T), dtype=torch.float32, device=q.device)
        dq = torch.empty_like(q)
        dk = torch.empty((T, Hkv, D), dtype=q.dtype, device=q.device)
        dv = torch.empty((T, Hkv, D), dtype=q.dtype, device=q.device)
        rc = _lib.kernels().b200_attn_bwd_ex(
            _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(o), _lib.ptr(do), _lib.ptr(lse), _lib.ptr(delta),
            _lib.ptr(dq_acc), _lib.ptr(dq), _lib.ptr(dk), _lib.ptr(dv), _lib.ptr(meta.bwd_tiles), ctypes.c_int(meta.n_bwd),
            ctypes.c_int(T), ctypes.c_int(T), ctypes.c_int(Hq), ctypes.c_int(Hkv), ctypes.c_longlong(k.stride(0)),
            ctypes.c_longlong(v.stride(0)), ctypes.c_longlong(dk.stride(0)), ctypes.c_longlong(dv.stride(0)),
            ctypes.c_float(ctx.scale), _lib.ptr(meta.key_exit), _lib.stream_ptr())
        _lib.check(rc, "b200_attn_bwd_ex")
        _lib.count_launch(3)
        return dq, dk, dv, None, None


def tree_attention(q, k, v, tree: PackedTree, meta: TreeMeta | None = None, scale: float | None = None):
    """Ancestor-masked attention over a packed tree batch: ``q [N, Hq, D]``, ``k/v [N, Hkv, D]``."""
    D = q.shape[-1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if _lib.use_cuda_kernels(q, k, v) and q.dtype == torch.bfloat16 and D == 128:
        k = k if (k.stride(2) == 1 and k.stride(1) == D) else k.contiguous()
        v = v if (v.stride(2) == 1 and v.stride(1) == D) else v.contiguous()
        return _TreeAttn.apply(q, k, v, meta or TreeMeta(tree, q.device), scale)
    return tree_attention_ref(q, k, v, tree, scale)
