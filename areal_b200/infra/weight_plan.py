"""Trainer → rollout weight transfer with re-sharding.

When the trainer runs data-parallel only, its flat weight buffer has the rollout engine's layout and the
transfer is a flat copy (``infra/dist_rollout.py``). Under tensor, pipeline or expert parallelism a trainer
rank holds *shards*: a slice of a fused projection, a stage's blocks, some experts. This module turns that
into a **push plan**: for every parameter shard a few strided copy segments ``(source offset in the
trainer's flat buffer) → (destination offset in the rollout engine's flat buffer)`` computed from the two
layouts, executed by one kernel that stores every segment into all destination buffers through NVLink peer
pointers (``b200_push_plan``). Ranks that hold identical data (data-parallel replicas, tensor-parallel peers
of a replicated tensor) share the work round-robin, so every destination byte is written exactly once and
no rank funnels the model.

The reference broadcasts full tensors from trainer rank 0 after gathering them (areal/engine/fsdp_engine.py:
1507-1597, per pipeline stage in areal/engine/megatron_engine.py:1640-1647); its experimental shard-to-shard
plans are areal/experimental/weight_update/awex/fsdp_adapter.py:118-170.
"""

from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass

import torch

from ..ops import _lib

PIECE_VECS = 1 << 18  # 4 MiB of 16-byte vectors per kernel block


@dataclass
class Segment:
    """``rows`` rows of ``row`` elements from ``src`` (row pitch ``src_pitch``) to ``dst`` (pitch ``dst_pitch``);
    offsets in elements of the respective flat buffer."""
    src: int
    dst: int
    rows: int
    row: int
    src_pitch: int
    dst_pitch: int


def rollout_layout(flat) -> dict[str, tuple[int, tuple[int, ...]]]:
    """``parameter name → (element offset, shape)`` of a flat buffer (the rollout engine publishes this)."""
    return {name: (off, shape) for name, (off, _, shape) in flat.named_offsets().items()}


def _global_name(name: str, layer_ids: list[int]) -> str:
    if name.startswith("layers."):
        _, idx, rest = name.split(".", 2)
        return f"layers.{layer_ids[int(idx)]}.{rest}"
    return name


def param_segments(name: str, shape: tuple[int, ...], full_shape: tuple[int, ...], cfg, tp_rank: int, tp: int,
                   ep_rank: int, ep: int, etp_rank: int = 0, etp: int = 1
                   ) -> list[tuple[int, int, int, int, int, int]] | None:
    """Segments of one parameter shard relative to the starts of the source and destination tensors, as
    ``(src, dst, rows, row, src_pitch, dst_pitch)``; ``None`` when this shard is a replica that the first
    tensor-parallel rank pushes."""
    n = math.prod(shape) if shape else 1
    if ep * etp > 1 and len(shape) == 3 and name.endswith(("mlp.gate_up", "mlp.down")):
        if etp == 1:
            return [(0, ep_rank * n, 1, n, n, n)]  # this rank's experts, a contiguous block of the stacked tensor
        # expert tensor parallelism: per expert, the slice of the gate rows and of the up rows (contiguous blocks
        # of whole rows), or a column block of the down projection (strided)
        e_loc, segs = shape[0], []
        per_src, per_dst = shape[1] * shape[2], full_shape[1] * full_shape[2]
        for e in range(e_loc):
            s0, d0 = e * per_src, (ep_rank * e_loc + e) * per_dst
            if name.endswith("mlp.gate_up"):
                half, full_half, cols = shape[1] // 2, full_shape[1] // 2, shape[2]
                segs.append((s0, d0 + etp_rank * half * cols, 1, half * cols, 0, 0))
                segs.append((s0 + half * cols, d0 + (full_half + etp_rank * half) * cols, 1, half * cols, 0, 0))
            else:
                segs.append((s0, d0 + etp_rank * shape[2], shape[1], shape[2], shape[2], full_shape[2]))
        return segs
    if tp == 1 or tuple(shape) == tuple(full_shape):
        if tp > 1 and tp_rank != 0:
            return None
        return [(0, 0, 1, n, n, n)]
    cols = shape[-1] if len(shape) > 1 else 1
    if name.endswith(("embed", "lm_head", "attn.q_b", "attn.kv_b", "attn.q")):  # contiguous blocks of rows
        return [(0, tp_rank * n, 1, n, n, n)]
    if name.endswith(("attn.qkv", "attn.qkv_bias")):
        nq, nk = cfg.q_size // tp, cfg.kv_size // tp
        qs, ks = cfg.q_size, cfg.kv_size
        return [(0, tp_rank * nq * cols, 1, nq * cols, 0, 0),
                (nq * cols, (qs + tp_rank * nk) * cols, 1, nk * cols, 0, 0),
                ((nq + nk) * cols, (qs + ks + tp_rank * nk) * cols, 1, nk * cols, 0, 0)]
    if name.endswith("mlp.gate_up"):
        half = shape[0] // 2
        full_half = full_shape[0] // 2
        return [(0, tp_rank * half * cols, 1, half * cols, 0, 0),
                (half * cols, (full_half + tp_rank * half) * cols, 1, half * cols, 0, 0)]
    if name.endswith(("attn.o", "mlp.down")):
        return [(0, tp_rank * cols, shape[0], cols, cols, full_shape[1])]
    raise NotImplementedError(f"no re-sharding rule for parameter {name} {tuple(shape)} -> {tuple(full_shape)}")


def build_plan(engine, layout: dict[str, tuple[int, tuple[int, ...]]]) -> dict[int, tuple[object, list[Segment]]]:
    """This trainer rank's share of the transfer: ``id(flat buffer) → (flat buffer, segments)``."""
    pctx = engine.pctx
    tp = pctx.tp_size if pctx is not None else 1
    tp_rank = pctx.tp_rank if pctx is not None else 0
    ep = pctx.ep_size if pctx is not None else 1
    ep_rank = pctx.ep_rank if pctx is not None else 0
    etp = pctx.etp_size if pctx is not None else 1
    etp_rank = pctx.etp_rank if pctx is not None else 0
    model, cfg = engine.model, engine.model_config
    layer_ids = list(getattr(model, "layer_ids", range(cfg.num_hidden_layers)))
    plans: dict[int, tuple[object, list[Segment]]] = {}
    flats = [f for f in (engine.weight_flat, getattr(engine, "flat_experts", None)) if f is not None]
    for f in flats:
        # ranks that hold the same bytes of this buffer share its segments round-robin
        share_rank, share_size = f.dp_rank, f.dp_world
        segs: list[Segment] = []
        k = 0
        for name, p, off, n in f.entries:
            gname = _global_name(name, layer_ids)
            if name == "embed" and not model.first_stage:
                continue  # the last pipeline stage's copy of a tied embedding: the first stage pushes it
            if gname not in layout:
                raise KeyError(f"the rollout engine has no parameter {gname}")
            dst_off, full_shape = layout[gname]
            rel = param_segments(name, tuple(p.shape), tuple(full_shape), cfg, tp_rank, tp, ep_rank, ep, etp_rank, etp)
            if rel is None:
                continue
            for s, d, rows, row, sp, dp in rel:
                if k % share_size == share_rank:
                    segs.append(Segment(off + s, dst_off + d, rows, row, sp or row, dp or row))
                k += 1
        plans[id(f)] = (f, segs)
    return plans


def _pieces(segs: list[Segment], itemsize: int) -> torch.Tensor:
    """Device-ready records in 16-byte units, large segments cut into pieces of at most ``PIECE_VECS``."""
    per = 16 // itemsize
    recs = []
    for g in segs:
        for v in (g.src, g.dst, g.row, g.src_pitch, g.dst_pitch):
            if v % per:
                raise ValueError(f"segment {g} is not aligned to 16 bytes")
        src, dst, row, sp, dp = g.src // per, g.dst // per, g.row // per, g.src_pitch // per, g.dst_pitch // per
        if g.rows == 1:
            for a in range(0, row, PIECE_VECS):
                m = min(PIECE_VECS, row - a)
                recs.append((src + a, dst + a, m, m, 1 | (m << 32)))
        else:
            step = max(PIECE_VECS // max(row, 1), 1)
            for r0 in range(0, g.rows, step):
                m = min(step, g.rows - r0)
                recs.append((src + r0 * sp, dst + r0 * dp, sp, dp, m | (row << 32)))
    return torch.tensor(recs, dtype=torch.int64).reshape(-1, 5)


class WeightPusher:
    """Executes this rank's plan against the destination buffers ``dst_ptrs`` (device pointers valid in this
    process: peer mappings of other ranks' rollout buffers, or the local buffer's own address)."""

    def __init__(self, engine, dst_ptrs: list[int], layout: dict[str, tuple[int, tuple[int, ...]]]):
        self.engine = engine
        self.n_dst = len(dst_ptrs)
        self.table = (ctypes.c_void_p * max(self.n_dst, 1))(*dst_ptrs)
        self.parts = []
        self.bytes = 0
        for f, segs in build_plan(engine, layout).values():
            item = f.flat.element_size()
            recs = _pieces(segs, item)
            self.bytes += sum(g.rows * g.row for g in segs) * item
            self.parts.append((f, recs.to(f.flat.device), recs.shape[0]))

    def push(self):
        lib = _lib.kernels()
        for f, recs, n in self.parts:
            if n == 0:
                continue
            rc = lib.b200_push_plan(self.table, ctypes.c_int(self.n_dst), _lib.ptr(f.flat), _lib.ptr(recs),
                                    ctypes.c_int(n), _lib.stream_ptr())
            _lib.check(rc, "b200_push_plan")
            _lib.count_launch()


def apply_plan_torch(plans: dict[int, tuple[object, list[Segment]]], dst: torch.Tensor):
    """PyTorch statement of the kernel for one destination buffer (CPU tests, gloo fallback)."""
    for f, segs in plans.values():
        for g in segs:
            for r in range(g.rows):
                dst[g.dst + r * g.dst_pitch: g.dst + r * g.dst_pitch + g.row].copy_(
                    f.flat[g.src + r * g.src_pitch: g.src + r * g.src_pitch + g.row])
