"""Context parallelism with gathered keys/values (zig-zag layout).

Every sequence (padded to a multiple of ``2 * cp * 128`` tokens) is cut into ``2 * cp`` chunks;
rank ``r`` keeps chunks ``r`` and ``2cp - 1 - r``, which balances causal work. Attention on a rank
uses its local queries against the keys/values of the whole sequence: K and V are all-gathered
(backward: reduce-scattered), brought into sequence order, and the varlen tcgen05 kernels run with
tile tables that give each local query block its causal extent in the gathered arrays. No rank
computes a score that another rank also computes.

:class:`CPLayout` owns the index bookkeeping (which packed tokens a rank holds, how gathered rows
map to sequence order, the tile tables); :func:`cp_attention_local` is the attention itself given
already-gathered K/V (this is what a single process can test by playing every rank in turn);
:func:`cp_attention` adds the collectives. Reference behaviour: zig-zag ``2*cp`` chunking of packed
sequences for ring / all-gather CP (areal/engine/megatron_utils/packed_context_parallel.py:14-185).
"""

from __future__ import annotations

import ctypes
import math

import numpy as np
import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops.attention import _BT, _QT, attention_ref

ALIGN = 128


class CPLayout:
    def __init__(self, seqlens: list[int], cp: int, rank: int, device="cpu"):
        """``seqlens``: true lengths of the packed sequences (each is padded up to ``2*cp*128``)."""
        self.cp, self.rank = cp, rank
        unit = 2 * cp * ALIGN
        self.padded = [(-(-L // unit)) * unit for L in seqlens]
        self.seqlens = list(seqlens)
        self.full_cu = np.concatenate([[0], np.cumsum(self.padded)]).astype(np.int64)
        self.T_full = int(self.full_cu[-1])
        # local rows: for every sequence chunk r then chunk 2cp-1-r
        local_idx = []
        self.chunks = []  # (seq, a, b, local_row_start) in sequence positions
        row = 0
        for s, Lp in enumerate(self.padded):
            c = Lp // (2 * cp)
            for ci in (rank, 2 * cp - 1 - rank):
                a, b = ci * c, (ci + 1) * c
                self.chunks.append((s, a, b, row))
                local_idx.append(np.arange(self.full_cu[s] + a, self.full_cu[s] + b))
                row += c
        self.T_local = row
        self.local_index = torch.from_numpy(np.concatenate(local_idx)).to(device)  # rows of the padded packed array
        # gathered (rank-major) row of every sequence-order row
        perm = np.empty(self.T_full, dtype=np.int64)
        for r in range(cp):
            row = 0
            for s, Lp in enumerate(self.padded):
                c = Lp // (2 * cp)
                for ci in (r, 2 * cp - 1 - r):
                    perm[self.full_cu[s] + ci * c: self.full_cu[s] + (ci + 1) * c] = r * self.T_local + row + np.arange(c)
                    row += c
        self.gather_to_seq = torch.from_numpy(perm).to(device)          # seq_order = gathered[gather_to_seq]
        inv = np.empty_like(perm)
        inv[perm] = np.arange(self.T_full)
        self.seq_to_gather = torch.from_numpy(inv).to(device)           # gathered = seq_order[seq_to_gather]
        self._tiles(device)

    def _tiles(self, device):
        fwd, bwd = [], [[], []]
        for n, (s, a, b, row) in enumerate(self.chunks):
            base = int(self.full_cu[s])
            kv_lim = self.seqlens[s]  # keys beyond the true length are padding
            for q0 in range(a, b, _QT):
                fwd.append((row + (q0 - a), _QT, base, min(kv_lim, q0 + _QT), q0, 0, 0, 0))
            which = n % 2  # lower / upper chunk of the sequence: two backward launches
            for k0 in range(0, min(b, kv_lim), _BT):
                # (kv_start, kv_len, kv_off, seq_start = local row of position 0, seq_len = b, q_begin = a)
                bwd[which].append((base + k0, min(_BT, kv_lim - k0), k0, row - a, b, a, 0, 0))
        fwd.sort(key=lambda t: -t[3])
        self.n_fwd = len(fwd)
        self.fwd_tiles = torch.tensor(fwd, dtype=torch.int32).reshape(-1, 8).to(device)
        self.bwd_tiles = []
        for lst in bwd:
            lst.sort(key=lambda t: -(t[4] - max(t[2], t[5])))
            self.bwd_tiles.append((len(lst), torch.tensor(lst, dtype=torch.int32).reshape(-1, 8).to(device)))

    def split(self, packed_padded: torch.Tensor) -> torch.Tensor:
        """Rows of a padded packed tensor ``[T_full, ...]`` that this rank holds."""
        return packed_padded.index_select(0, self.local_index.to(packed_padded.device))

    def pad_packed(self, x: torch.Tensor) -> torch.Tensor:
        """``[sum(seqlens), ...]`` → ``[T_full, ...]`` with zero rows after every sequence."""
        out = x.new_zeros((self.T_full,) + tuple(x.shape[1:]))
        o = 0
        for s, L in enumerate(self.seqlens):
            out[int(self.full_cu[s]):int(self.full_cu[s]) + L] = x[o:o + L]
            o += L
        return out


def _ref_local(q_loc, k_full, v_full, lay: CPLayout, scale):
    """PyTorch restatement: local queries against the sequence-ordered gathered keys."""
    out = torch.zeros_like(q_loc, dtype=torch.float32)
    g = q_loc.shape[1] // k_full.shape[1]
    for (s, a, b, row) in lay.chunks:
        base, L = int(lay.full_cu[s]), lay.seqlens[s]
        kv = min(b, L)
        if kv == 0:
            continue
        qs = q_loc[row:row + (b - a)].float().transpose(0, 1)
        ks = k_full[base:base + kv].float().transpose(0, 1).repeat_interleave(g, 0)
        vs = v_full[base:base + kv].float().transpose(0, 1).repeat_interleave(g, 0)
        att = qs @ ks.transpose(1, 2) * scale
        qpos = torch.arange(a, b, device=q_loc.device)[:, None]
        kpos = torch.arange(kv, device=q_loc.device)[None, :]
        att = att.masked_fill(kpos > qpos, float("-inf")).softmax(-1)
        out[row:row + (b - a)] = (att @ vs).transpose(0, 1)
    return out.to(q_loc.dtype)


class _CPAttnLocal(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k_full, v_full, lay: CPLayout, scale):
        T, Hq, D = q.shape
        Hkv = k_full.shape[1]
        q, k_full, v_full = q.contiguous(), k_full.contiguous(), v_full.contiguous()
        o = torch.empty_like(q)
        lse = torch.empty((Hq, T), dtype=torch.float32, device=q.device)
        rc = _lib.kernels().b200_attn_fwd_ex(
            _lib.ptr(q), _lib.ptr(k_full), _lib.ptr(v_full), _lib.ptr(o), _lib.ptr(lse), _lib.ptr(lay.fwd_tiles),
            ctypes.c_int(lay.n_fwd), ctypes.c_int(T), ctypes.c_int(lay.T_full), ctypes.c_int(Hq), ctypes.c_int(Hkv),
            ctypes.c_longlong(q.stride(0)), ctypes.c_longlong(k_full.stride(0)), ctypes.c_longlong(v_full.stride(0)),
            ctypes.c_float(scale), None, _lib.stream_ptr())
        _lib.check(rc, "b200_attn_fwd_ex")
        _lib.count_launch()
        ctx.save_for_backward(q, k_full, v_full, o, lse)
        ctx.lay, ctx.scale = lay, scale
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse = ctx.saved_tensors
        lay: CPLayout = ctx.lay
        T, Hq, D = q.shape
        Hkv = k.shape[1]
        do = do.contiguous()
        dq_acc = torch.zeros((T, Hq, D), dtype=torch.float32, device=q.device)
        delta = torch.empty((Hq, T), dtype=torch.float32, device=q.device)
        dq = torch.empty_like(q)
        dks, dvs = [], []
        for i, (n, tiles) in enumerate(lay.bwd_tiles):
            dk = torch.zeros((lay.T_full, Hkv, D), dtype=q.dtype, device=q.device)
            dv = torch.zeros_like(dk)
            last = i == len(lay.bwd_tiles) - 1
            rc = _lib.kernels().b200_attn_bwd_ex(
                _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(o), _lib.ptr(do), _lib.ptr(lse), _lib.ptr(delta),
                _lib.ptr(dq_acc), _lib.ptr(dq) if last else None, _lib.ptr(dk), _lib.ptr(dv), _lib.ptr(tiles),
                ctypes.c_int(n), ctypes.c_int(T), ctypes.c_int(lay.T_full), ctypes.c_int(Hq), ctypes.c_int(Hkv),
                ctypes.c_longlong(k.stride(0)), ctypes.c_longlong(v.stride(0)), ctypes.c_longlong(dk.stride(0)),
                ctypes.c_longlong(dv.stride(0)), ctypes.c_float(ctx.scale), None, _lib.stream_ptr())
            _lib.check(rc, "b200_attn_bwd_ex")
            _lib.count_launch(3)
            dks.append(dk)
            dvs.append(dv)
        return dq, dks[0] + dks[1], dvs[0] + dvs[1], None, None


def cp_attention_local(q_loc, k_full, v_full, lay: CPLayout, scale: float | None = None):
    """``q_loc [T_local, Hq, D]`` (this rank's zig-zag rows) against sequence-ordered ``k_full / v_full
    [T_full, Hkv, D]``; differentiable in all three."""
    D = q_loc.shape[-1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if _lib.use_cuda_kernels(q_loc, k_full, v_full) and q_loc.dtype == torch.bfloat16 and D == 128:
        return _CPAttnLocal.apply(q_loc, k_full, v_full, lay, scale)
    return _ref_local(q_loc, k_full, v_full, lay, scale)


class _GatherKV(torch.autograd.Function):
    """All-gather rows over the cp group and reorder to sequence order; backward: the reverse
    reorder and a reduce-scatter (each rank holds a partial gradient for every key)."""

    @staticmethod
    def forward(ctx, x, group, lay: CPLayout):
        ctx.group, ctx.lay = group, lay
        out = torch.empty((lay.cp * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        if x.is_cuda:
            dist.all_gather_into_tensor(out, x.contiguous(), group=group)
        else:
            dist.all_gather(list(out.chunk(lay.cp, 0)), x.contiguous(), group=group)
        return out.index_select(0, lay.gather_to_seq.to(x.device))

    @staticmethod
    def backward(ctx, g):
        lay = ctx.lay
        g = g.index_select(0, lay.seq_to_gather.to(g.device)).contiguous()
        n = g.shape[0] // lay.cp
        if g.is_cuda:
            out = torch.empty((n,) + tuple(g.shape[1:]), dtype=g.dtype, device=g.device)
            dist.reduce_scatter_tensor(out, g, group=ctx.group)
        else:
            dist.all_reduce(g, group=ctx.group)
            out = g[lay.rank * n:(lay.rank + 1) * n].contiguous()
        return out, None, None


def cp_attention(q_loc, k_loc, v_loc, lay: CPLayout, group, scale: float | None = None):
    k_full = _GatherKV.apply(k_loc, group, lay)
    v_full = _GatherKV.apply(v_loc, group, lay)
    return cp_attention_local(q_loc, k_full, v_full, lay, scale)


def full_attention_reference(q, k, v, seqlens, scale=None):
    """Ordinary causal attention over the (unpadded) packed batch; the oracle of the tests."""
    cu = [0]
    for L in seqlens:
        cu.append(cu[-1] + L)
    return attention_ref(q, k, v, cu, scale)
