"""Expert parallelism for MoE layers over NVLink peer memory.

Experts are split over the ``P`` ranks of the ep group. One MoE layer is four phases; the first
and last run on every rank for ITS tokens, the middle ones on every rank for ITS experts:

1. ``sort``     – local stable sort of the (token, choice) copies by global expert
                  (``ops.moe.sort_by_expert``) → per-expert counts;
   counts are all-gathered (tiny) and ``plan`` turns them, on the device, into the row at which
   each copy lands in its owner's padded expert-sorted buffer, plus the owner-side tile table;
2. ``dispatch`` – one kernel stores every token row straight into the owners' buffers (peer
                  stores), together with the routing weight of the row;
3. ``experts``  – the owner zero-fills the padding rows and runs the grouped GEMMs in place;
4. ``combine``  – one kernel pulls the result rows back from the owners and forms the weighted
                  sum per token (peer loads).

The backward pass is the same four phases with gradients: dispatch ``dout``, owner-side grouped
dgrad / wgrad, combine the input gradients, and pull the per-copy routing-weight gradients.
Between phases the ranks meet at device-side barriers (``SymmBarrier``); the host never reads a
count. :class:`EPRank` holds one rank's buffers and implements the phases against explicit peer
pointer tables, which also lets a single process drive several virtual ranks on one GPU (how the
GPU test exercises it); :func:`ep_moe_forward` strings the phases together for real ranks.

Replaces the reference's count all-to-all + ``tolist()`` host sync + token all-to-all
(areal/experimental/models/archon/expert_parallel.py:70-262).
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops import moe as M


@dataclass
class EPPlan:
    send_base: torch.Tensor
    local: M.ExpertSort  # owner-side view: tile table, segment starts, totals (counts field)


def _ptr_array(ptrs: list[int], device) -> torch.Tensor:
    return torch.tensor(ptrs, dtype=torch.int64, device=device)


class EPRank:
    """Buffers of one ep rank. ``cap`` rows bound what this rank can receive for its experts."""

    def __init__(self, rank: int, world: int, num_experts: int, hidden: int, cap_rows: int, device, alloc=None):
        assert num_experts % world == 0
        self.rank, self.world, self.E, self.H = rank, world, num_experts, hidden
        self.el = num_experts // world
        self.cap = (cap_rows + 127) // 128 * 128 + self.el * 128
        self.device = device
        alloc = alloc or (lambda nbytes: torch.empty(nbytes, dtype=torch.uint8, device=device))
        self._raw = [alloc(self.cap * hidden * 2), alloc(self.cap * hidden * 2), alloc(self.cap * 4), alloc(self.cap * 4)]
        self.xbuf = self._raw[0].view(torch.bfloat16).view(self.cap, hidden)   # dispatched rows (x or dout)
        self.ybuf = self._raw[1].view(torch.bfloat16).view(self.cap, hidden)   # rows to be pulled (y or dxs)
        self.row_w = self._raw[2].view(torch.float32)                           # routing weight of each row
        self.s_out = self._raw[3].view(torch.float32)                           # <dout_row, y_row>
        self.peer_x = self.peer_y = self.peer_w = self.peer_s = None

    def pointers(self) -> tuple[int, int, int, int]:
        return self.xbuf.data_ptr(), self.ybuf.data_ptr(), self.row_w.data_ptr(), self.s_out.data_ptr()

    def connect(self, all_pointers: list[tuple[int, int, int, int]]):
        """``all_pointers[d]``: the four buffer addresses of rank ``d`` as seen from this process."""
        cols = list(zip(*all_pointers))
        self.peer_x, self.peer_y, self.peer_w, self.peer_s = (_ptr_array(list(c), self.device) for c in cols)

    # ---------------------------------------------------------------- phases
    def plan(self, counts_all: torch.Tensor) -> EPPlan:
        """``counts_all [P, E]`` int32 on the device (every rank's per-expert copy counts)."""
        dev = self.device
        ints = lambda n: torch.empty(n, dtype=torch.int32, device=dev)
        send_base, prow0, total, tiles, num_vm = ints(self.E), ints(self.el + 1), ints(self.el), ints(self.cap // 128), ints(1)
        rc = _lib.kernels().b200_ep_plan(_lib.ptr(counts_all.contiguous()), ctypes.c_int(self.rank),
                                         ctypes.c_int(self.world), ctypes.c_int(self.E), _lib.ptr(send_base),
                                         _lib.ptr(prow0), _lib.ptr(total), _lib.ptr(tiles), _lib.ptr(num_vm),
                                         _lib.stream_ptr())
        _lib.check(rc, "b200_ep_plan")
        _lib.count_launch()
        local = M.ExpertSort(n=0, k=1, num_experts=self.el, max_rows=self.cap, dest=None, src_of=None, counts=total,
                             prow0=prow0, tile_expert=tiles, num_vm=num_vm)
        return EPPlan(send_base, local)

    def dispatch(self, x: torch.Tensor, idx: torch.Tensor, w: torch.Tensor | None, s: M.ExpertSort, plan: EPPlan):
        """Stores this rank's token rows into the owners' ``xbuf`` (and ``row_w``); returns the
        row of every copy ``[T*k]``."""
        n = s.n
        copy_row = torch.empty(n, dtype=torch.int32, device=self.device)
        x = x if x.stride(1) == 1 else x.contiguous()
        if _lib.checked():
            _lib.check_operand("ep_dispatch.idx", idx, torch.int32, None, align=4)
            _lib.check_index("ep_dispatch.expert_ids", idx, self.el * self.world)
        rc = _lib.kernels().b200_ep_dispatch(_lib.ptr(x), ctypes.c_longlong(x.stride(0)), _lib.ptr(idx), _lib.ptr(w),
                                             _lib.ptr(s.dest), _lib.ptr(s.prow0), _lib.ptr(plan.send_base),
                                             ctypes.c_int(n), ctypes.c_int(s.k), ctypes.c_int(self.H),
                                             ctypes.c_int(self.el), ctypes.c_int(self.cap), _lib.ptr(self.peer_x),
                                             _lib.ptr(self.peer_w), _lib.ptr(copy_row), _lib.stream_ptr())
        _lib.check(rc, "b200_ep_dispatch")
        _lib.count_launch()
        return copy_row

    def zero_padding(self, plan: EPPlan, with_weights: bool = True):
        rc = _lib.kernels().b200_ep_zero_pad(_lib.ptr(self.xbuf), _lib.ptr(self.row_w if with_weights else None),
                                             _lib.ptr(plan.local.prow0), _lib.ptr(plan.local.counts),
                                             ctypes.c_int(self.el), ctypes.c_int(self.H), _lib.stream_ptr())
        _lib.check(rc, "b200_ep_zero_pad")
        _lib.count_launch()

    def experts_forward(self, plan: EPPlan, gate_up: torch.Tensor, down: torch.Tensor):
        """Grouped SwiGLU MLP over the received rows; the result lands in ``ybuf``. Returns what
        the backward needs (copies: the symmetric buffers are reused by the next layer)."""
        self.zero_padding(plan)
        ls = plan.local
        h1 = M.grouped_gemm(self.xbuf, gate_up, ls)
        a = M._swiglu_raw(h1)
        _grouped_into(a, down, ls, self.ybuf)
        return dict(xs=self.xbuf.clone(), h1=h1, y=self.ybuf.clone(), row_w=self.row_w.clone(), plan=plan)

    def combine(self, idx: torch.Tensor, copy_row: torch.Tensor, w: torch.Tensor | None, T: int, k: int):
        out = torch.empty((T, self.H), dtype=torch.bfloat16, device=self.device)
        rc = _lib.kernels().b200_ep_combine(_lib.ptr(self.peer_y), _lib.ptr(idx), _lib.ptr(copy_row), _lib.ptr(w),
                                            ctypes.c_int(T), ctypes.c_int(k), ctypes.c_int(self.H),
                                            ctypes.c_int(self.el), _lib.ptr(out), _lib.stream_ptr())
        _lib.check(rc, "b200_ep_combine")
        _lib.count_launch()
        return out

    def experts_backward(self, saved: dict, gate_up: torch.Tensor, down: torch.Tensor):
        """``xbuf`` holds the dispatched ``dout`` rows. Leaves ``dxs`` in ``ybuf`` and
        ``<dout_row, y_row>`` in ``s_out``; returns ``(d_gate_up, d_down)`` (None when the
        parameters carry ``main_grad``)."""
        plan = saved["plan"]
        ls = plan.local
        self.zero_padding(plan, with_weights=False)
        lib = _lib.kernels()
        # s = <dout, y> per row, then dy = w_row * dout in place
        rc = lib.b200_rowdot_scale(_lib.ptr(self.xbuf), _lib.ptr(saved["y"]), _lib.ptr(saved["row_w"]),
                                   _lib.ptr(ls.num_vm), ctypes.c_int(self.cap), ctypes.c_int(self.H),
                                   _lib.ptr(self.s_out), _lib.stream_ptr())
        _lib.check(rc, "b200_rowdot_scale")
        _lib.count_launch()
        dy = self.xbuf
        a = M._swiglu_raw(saved["h1"])
        da = M.grouped_gemm(dy, down, ls, transpose_w=False)
        d_down = M._wgrad_into(down, dy, a, ls)
        dh1 = M._swiglu_bwd_raw(da, saved["h1"])
        d_gate_up = M._wgrad_into(gate_up, dh1, saved["xs"], ls)
        _grouped_into(dh1, gate_up, ls, self.ybuf, transpose_w=False)
        return d_gate_up, d_down

    def pull_weight_grads(self, idx: torch.Tensor, copy_row: torch.Tensor):
        n = idx.numel()
        vals = torch.empty(n, dtype=torch.float32, device=self.device)
        rc = _lib.kernels().b200_ep_pull_scalar(_lib.ptr(self.peer_s), _lib.ptr(idx), _lib.ptr(copy_row), ctypes.c_int(n),
                                                ctypes.c_int(self.el), _lib.ptr(vals), _lib.stream_ptr())
        _lib.check(rc, "b200_ep_pull_scalar")
        _lib.count_launch()
        return vals


def _grouped_into(a, w, ls, out, transpose_w=True):
    """Grouped GEMM writing into a caller-owned (symmetric) buffer."""
    E = w.shape[0]
    K = a.shape[1]
    N = w.shape[1] if transpose_w else w.shape[2]
    assert out.shape[1] == N
    rc = _lib.kernels().b200_gemm_grouped(_lib.ptr(a), _lib.ptr(w), _lib.ptr(out), _lib.ptr(ls.tile_expert),
                                          _lib.ptr(ls.num_vm), ctypes.c_int(ls.max_rows), ctypes.c_int(E),
                                          ctypes.c_int(N), ctypes.c_int(K), ctypes.c_int(0 if transpose_w else 1),
                                          _lib.stream_ptr())
    _lib.check(rc, "b200_gemm_grouped")
    _lib.count_launch()


# --------------------------------------------------------------------------- real ranks


class EPGroupState:
    """One per model: the symmetric buffers of this rank, mapped on every peer of the ep group."""

    def __init__(self, group, num_experts: int, hidden: int, cap_rows: int, device=None):
        from .symm_mem import SymmBarrier, SymmBuffer

        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        dev = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        bufs: list = []

        def alloc(nbytes):
            b = SymmBuffer(nbytes, group, dev)
            bufs.append(b)
            return b.tensor(torch.uint8, nbytes)

        self.me = EPRank(self.rank, self.world, num_experts, hidden, cap_rows, dev, alloc=alloc)
        self._bufs = bufs
        self.me.connect([tuple(b.peer_ptrs[d] for b in bufs) for d in range(self.world)])
        self.barrier = SymmBarrier(group, dev)

    def all_counts(self, counts: torch.Tensor) -> torch.Tensor:
        out = torch.empty((self.world, counts.numel()), dtype=counts.dtype, device=counts.device)
        dist.all_gather_into_tensor(out, counts.contiguous(), group=self.group)
        return out


class _EPMoE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, idx, w, gate_up, down, st: EPGroupState):
        me = st.me
        T, k = idx.shape
        idx = idx.to(torch.int32).contiguous()
        w32 = w.float().contiguous()
        s = M.sort_by_expert(idx, me.E)
        plan = me.plan(st.all_counts(s.counts))
        st.barrier.sync()  # every peer is done reading my buffers from the previous layer
        copy_row = me.dispatch(x, idx.view(-1), w32.view(-1), s, plan)
        st.barrier.sync()  # all rows have landed
        saved = me.experts_forward(plan, gate_up, down)
        st.barrier.sync()  # every owner's results are complete
        out = me.combine(idx.view(-1), copy_row, w32.view(-1), T, k)
        ctx.st, ctx.saved, ctx.s, ctx.copy_row, ctx.idx = st, saved, s, copy_row, idx
        ctx.save_for_backward(w32, gate_up, down)
        ctx.w_dtype = w.dtype
        return out

    @staticmethod
    def backward(ctx, dout):
        st, me = ctx.st, ctx.st.me
        w32, gate_up, down = ctx.saved_tensors
        T, k = ctx.idx.shape
        idx = ctx.idx.view(-1)
        st.barrier.sync()
        me.dispatch(dout.contiguous(), idx, None, ctx.s, ctx.saved["plan"])
        st.barrier.sync()
        d_gate_up, d_down = me.experts_backward(ctx.saved, gate_up, down)
        st.barrier.sync()
        dx = me.combine(idx, ctx.copy_row, None, T, k)
        dw = me.pull_weight_grads(idx, ctx.copy_row).view(T, k).to(ctx.w_dtype)
        return dx, None, dw, d_gate_up, d_down, None


def ep_moe_forward(x, idx, w, gate_up_local, down_local, st):
    """``x [T,H]`` (this rank's tokens), ``idx/w [T,k]`` over GLOBAL expert ids, local expert weights
    ``[E/P, 2I, H]`` / ``[E/P, H, I]``. ``st`` is an :class:`EPGroupState` (CUDA) or a plain process
    group (CPU / gloo: tokens are all-gathered, every rank applies its experts to all of them and
    the partial outputs are summed back; slower, same result)."""
    if isinstance(st, EPGroupState):
        return _EPMoE.apply(x.contiguous(), idx, w, gate_up_local, down_local, st)
    return _ep_moe_gathered(x, idx, w, gate_up_local, down_local, st)


def _gather_var(t: torch.Tensor, group) -> tuple[torch.Tensor, list[int]]:
    """Concatenation of every rank's rows and the row counts (tensor collectives: counts first, then the rows
    padded to the largest count)."""
    P = dist.get_world_size(group)
    t = t.detach().contiguous()
    n = torch.tensor([t.shape[0]], dtype=torch.int64, device=t.device)
    ns = [torch.empty_like(n) for _ in range(P)]
    dist.all_gather(ns, n, group=group)
    sizes = [int(v) for v in ns]
    m = max(sizes)
    if t.shape[0] < m:
        t = torch.cat((t, t.new_zeros((m - t.shape[0],) + tuple(t.shape[1:]))), 0)
    parts = [torch.empty_like(t) for _ in range(P)]
    dist.all_gather(parts, t, group=group)
    return torch.cat([p[:k] for p, k in zip(parts, sizes)], 0), sizes


class _GatherVar(torch.autograd.Function):
    """Concatenates every rank's rows (row counts may differ); backward: sum over ranks, keep own rows."""

    @staticmethod
    def forward(ctx, t, group):
        full, sizes = _gather_var(t, group)
        ctx.group, ctx.sizes = group, sizes
        return full

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous().clone()
        dist.all_reduce(g, group=ctx.group)
        r = dist.get_rank(ctx.group)
        a = sum(ctx.sizes[:r])
        return g[a:a + ctx.sizes[r]], None


class _ReduceSlice(torch.autograd.Function):
    """Sum over ranks, keep own rows; backward: concatenate every rank's gradient rows."""

    @staticmethod
    def forward(ctx, t, group, sizes):
        t = t.contiguous().clone()
        dist.all_reduce(t, group=group)
        r = dist.get_rank(group)
        a = sum(sizes[:r])
        ctx.group = group
        return t[a:a + sizes[r]]

    @staticmethod
    def backward(ctx, g):
        full, _ = _gather_var(g.contiguous(), ctx.group)
        return full, None, None


def _ep_moe_gathered(x, idx, w, gate_up_local, down_local, group):
    P, r = dist.get_world_size(group), dist.get_rank(group)
    el = gate_up_local.shape[0]
    x_all = _GatherVar.apply(x, group)
    w_all = _GatherVar.apply(w.float(), group)
    idx_all, sizes = _gather_var(idx, group)
    local = (idx_all >= r * el) & (idx_all < (r + 1) * el)
    part = M.moe_experts_ref(x_all, torch.where(local, idx_all - r * el, torch.zeros_like(idx_all)),
                             w_all * local, gate_up_local, down_local)
    return _ReduceSlice.apply(part, group, sizes).to(x.dtype)


def etp_moe_forward(x, idx, w, group, experts):
    """Expert tensor parallelism around ``experts(x, idx, w)`` (the local or expert-parallel mixture over this
    rank's SLICE of the expert weights, whose output is therefore a partial sum): the ranks of ``group`` pool
    their tokens with the routing each computed for its own, apply their slices to all of them and get back the
    sum of the partial outputs for their own rows. Row counts may differ between ranks."""
    x_all = _GatherVar.apply(x, group)
    w_all = _GatherVar.apply(w.float(), group)
    idx_all, sizes = _gather_var(idx, group)
    part = experts(x_all, idx_all, w_all.to(w.dtype))
    return _ReduceSlice.apply(part, group, sizes).to(x.dtype)
