"""``torch.distributed.checkpoint`` (DCP) state of the train engine.

The engine keeps weights, fp32 master weights and Adam moments in flat buffers that are sharded by
flat offset over the data-parallel (x Ulysses) group, so a rank's shard starts and ends in the middle of
parameters. DCP wants named tensors with box-shaped chunks. :class:`ShardedView` bridges the two: it is a
tensor subclass that stands for ONE named tensor of the checkpoint (an HF-named weight, e.g.
``model.layers.3.self_attn.q_proj.weight``, at its full, unsharded shape) of which this rank holds a
contiguous *flat range*; the range is cut into at most ``2 * ndim - 1`` boxes (partial first row, block of
full rows, partial last row, recursively), each a view into the engine's own buffer, and announced to DCP
through its checkpointable protocol (``__create_write_items__`` / ``__create_chunk_list__`` /
``__get_tensor_shard__``). DCP then reshards on load by intersecting saved and wanted boxes, which is what
makes a checkpoint written at one data-parallel size loadable at another, and what makes the model part of a
checkpoint written by FSDP2 (``Shard(0)`` DTensors under the same names) loadable here.

Layout of a checkpoint (flattened keys), the same top level as the reference's ``DCPState``
(areal/engine/fsdp_utils/checkpoint.py:19-69, used by areal/engine/fsdp_engine.py:1668-1693):

* ``dcp.model.<hf name>``: weights in the training dtype;
* ``dcp.optim.state.<hf name>.exp_avg`` / ``.exp_avg_sq`` / ``.master``: Adam moments and the fp32 master
  copy (for ``adam_bf16`` ``master`` is the Kahan compensation);
* ``dcp.optim.meta``: step counters and the optimizer kind;
* ``dcp.rng.rank<r>``: CPU (and CUDA) generator state of global rank ``r`` (restored only when the world
  size is unchanged).

Tensor-parallel shards sit at their offset along the split dimension, pipeline stages and expert-parallel
ranks own disjoint names, and every rank writes only what overlaps its own flat shard, so no tensor is
written twice and none is gathered.
"""

from __future__ import annotations

import io
import math
from typing import Any, Iterator

import torch
import torch.distributed as dist
from torch.distributed.checkpoint.metadata import ChunkStorageMetadata, MetadataIndex, TensorProperties
from torch.distributed.checkpoint.planner import TensorWriteData, WriteItem, WriteItemType
from torch.distributed.checkpoint.stateful import Stateful


def flat_range_boxes(shape: tuple[int, ...], a: int, b: int) -> list[tuple[tuple[int, ...], tuple[int, ...], int]]:
    """Cuts the row-major flat range ``[a, b)`` of a tensor of ``shape`` into boxes, each contiguous in
    memory. Returns ``(offsets, sizes, flat_start)`` per box, in increasing flat order."""
    out: list[tuple[tuple[int, ...], tuple[int, ...], int]] = []
    if not shape:  # a scalar
        return [((), (), 0)] if b > a else []

    def rec(dims: tuple[int, ...], lo: int, hi: int, prefix: tuple[int, ...], base: int):
        if lo >= hi:
            return
        if len(dims) == 1:
            out.append((prefix + (lo,), (1,) * len(prefix) + (hi - lo,), base + lo))
            return
        inner = math.prod(dims[1:])
        i0, r0 = divmod(lo, inner)
        i1, r1 = divmod(hi, inner)
        if i0 == i1:
            rec(dims[1:], r0, r1, prefix + (i0,), base + i0 * inner)
            return
        if r0 > 0:
            rec(dims[1:], r0, inner, prefix + (i0,), base + i0 * inner)
            i0 += 1
        if i1 > i0:
            out.append((prefix + (i0,) + (0,) * (len(dims) - 1), (1,) * len(prefix) + (i1 - i0,) + tuple(dims[1:]),
                        base + i0 * inner))
        if r1 > 0:
            rec(dims[1:], 0, r1, prefix + (i1,), base + i1 * inner)

    rec(tuple(shape), a, b, (), 0)
    return out


class ShardedView(torch.Tensor):
    """One named checkpoint tensor of ``global_shape`` of which this rank holds some boxes, each a view
    into a buffer of the engine. It has no storage of its own and supports no operators: DCP only asks it
    for its chunks and for the tensor behind a chunk."""

    @staticmethod
    def __new__(cls, global_shape, dtype, device, boxes):
        r = torch.Tensor._make_wrapper_subclass(cls, tuple(global_shape), dtype=dtype, device=device,
                                                requires_grad=False)
        r._boxes = list(boxes)  # (global offsets, sizes, local tensor of that size)
        return r

    @classmethod
    def __torch_dispatch__(cls, func, types, args=(), kwargs=None):
        raise NotImplementedError(f"ShardedView is a checkpoint handle, not an operand ({func})")

    def __repr__(self):  # the default repr would dispatch
        return f"ShardedView(shape={tuple(self.shape)}, dtype={self.dtype}, boxes={len(self._boxes)})"

    # --- torch.distributed._checkpointable protocol
    def __create_write_items__(self, fqn: str, obj: Any):
        size = torch.Size(self.shape)
        items = []
        for off, sz, t in self._boxes:
            items.append(WriteItem(
                index=MetadataIndex(fqn, torch.Size(off)), type=WriteItemType.SHARD,
                tensor_data=TensorWriteData(chunk=ChunkStorageMetadata(offsets=torch.Size(off), sizes=torch.Size(sz)),
                                            properties=TensorProperties.create_from_tensor(t), size=size)))
        return items

    def __create_chunk_list__(self):
        return [ChunkStorageMetadata(offsets=torch.Size(off), sizes=torch.Size(sz)) for off, sz, _ in self._boxes]

    def __get_tensor_shard__(self, index: MetadataIndex) -> torch.Tensor:
        if index.index is not None and index.index < len(self._boxes) and \
                torch.Size(self._boxes[index.index][0]) == index.offset:
            return self._boxes[index.index][2]
        for off, _, t in self._boxes:
            if torch.Size(off) == index.offset:
                return t
        raise ValueError(f"no local box at offset {index.offset} of {index.fqn}")


def _flat_of(view: torch.Tensor, flats) -> tuple[Any, int] | None:
    """The flat buffer a parameter view lives in and its element offset there."""
    p = view.data_ptr()
    for f in flats:
        base = f.flat.data_ptr()
        item = f.flat.element_size()
        if base <= p < base + f.numel * item and view.dtype == f.flat.dtype:
            return f, (p - base) // item
    return None


class EngineDCPState(Stateful):
    """``Stateful`` wrapper over a ``B200TrainEngine`` for ``dcp.save`` / ``dcp.load`` (the reference's
    ``DCPState``). ``state_dict()`` returns handles into the engine's own buffers; loading fills them in
    place and ``load_state_dict`` then republishes the weights to every rank of the shard group."""

    def __init__(self, engine, with_optim: bool = True, available: set[str] | None = None, prefix: str = "dcp.",
                 with_model: bool = True):
        self.e = engine
        self.with_model = with_model  # False: optimizer state only (beside an HF-format weight checkpoint)
        self.with_optim = with_optim and engine.optimizer is not None
        # keys present in the checkpoint being loaded (None when saving): optional parts that the checkpoint
        # does not hold are left out of the request instead of failing the load
        self.available = available
        self.prefix = prefix
        self.loaded_optim_meta: dict | None = None

    # ------------------------------------------------------------------ names
    def _named_views(self, for_load: bool) -> Iterator[tuple[str, Any, int, tuple[int, ...], int | None]]:
        """``(hf name, flat buffer, flat offset, local shape, tp dim)`` of every stored tensor."""
        e = self.e
        model = e.model
        flats = [f for f in (e.flat, getattr(e, "flat_base", None), getattr(e, "flat_experts", None)) if f is not None]
        covered: dict[int, list[tuple[int, int]]] = {id(f): [] for f in flats}
        views = list(model.to_hf_local())
        tied_copy = None
        if model.embed is not None and not model.first_stage:
            # the last stage's copy of a tied embedding is written by the first stage only, read by both
            lm = getattr(model, "_LM", None)
            tied_copy = (lm + "embed_tokens.weight") if lm else "model.embed_tokens.weight"
            views.append((tied_copy, model.embed))
        for name, v in views:
            if not v.is_contiguous():
                continue
            hit = _flat_of(v, flats)
            if hit is None:
                continue
            f, off = hit
            covered[id(f)].append((off, off + v.numel()))
            if name == tied_copy and not for_load:
                continue
            spec = model.shard_spec(name) if hasattr(model, "shard_spec") else None
            yield name, f, off, tuple(v.shape), (None if spec is None else spec[:3])
        tp = e.pctx.tp_size if e.pctx is not None else 1
        for f in flats:
            spans = sorted(covered[id(f)])
            for pname, p, o, n in f.entries:
                got = sum(min(b, o + n) - max(a, o) for a, b in spans if a < o + n and b > o)
                if got >= n:
                    continue
                spec = None
                if tp > 1:
                    from ..parallel.tensor_parallel import is_tp_replicated, lora_tp_dim

                    if not is_tp_replicated(pname):
                        d = lora_tp_dim(pname) if ".lora_" in pname else None
                        if d is None:
                            raise NotImplementedError(
                                f"parameter {pname} has no checkpoint name under tensor parallelism")
                        spec = (d, e.pctx.tp_rank, tp)  # a low-rank adapter factor split over the tp group
                if pname.startswith("layers.") and hasattr(model, "layer_ids"):
                    # a pipeline stage numbers its blocks from 0: the checkpoint name carries the global index
                    _, idx, rest = pname.split(".", 2)
                    pname = f"layers.{model.layer_ids[int(idx)]}.{rest}"
                yield "_native." + pname, f, o, tuple(p.shape), spec

    def _handle(self, f, off: int, shape: tuple[int, ...], tp_dim: int | None, buf: torch.Tensor, buf_start: int,
                write: bool) -> ShardedView | None:
        """Handle of the part of ``[off, off + numel)`` (flat coordinates of ``f``) that lies in
        ``[buf_start, buf_start + len(buf))``; ``buf`` is the tensor holding that window."""
        e = self.e
        n = math.prod(shape) if shape else 1
        lo, hi = max(off, buf_start), min(off + n, buf_start + buf.numel())
        tp = e.pctx.tp_size if e.pctx is not None else 1
        tp_rank = e.pctx.tp_rank if e.pctx is not None else 0
        gshape = list(shape)
        shift = [0] * len(shape)
        if tp_dim is not None:
            # ``tp_dim`` is ``(dimension, rank, size)`` of the split over the tensor-parallel group (dense
            # projections) or the expert-tensor-parallel group (one expert's projections)
            dim, srank, ssize = tp_dim
            gshape[dim] *= ssize
            shift[dim] = srank * shape[dim]
        elif write and tp > 1 and tp_rank != 0 and f is not getattr(e, "flat_experts", None):
            # replicated over the tensor-parallel group: its first rank writes (expert tensors are not replicated:
            # under the hybrid layout every tensor-parallel rank holds other experts)
            lo = hi = 0
        boxes = []
        for box_off, box_sz, start in flat_range_boxes(shape, lo - off, hi - off) if hi > lo else []:
            t = buf[off + start - buf_start: off + start - buf_start + math.prod(box_sz)].view(box_sz)
            boxes.append((tuple(o + s for o, s in zip(box_off, shift)), box_sz, t))
        return ShardedView(tuple(gshape), buf.dtype, buf.device, boxes)

    # ------------------------------------------------------------- Stateful
    def _build(self, write: bool) -> dict[str, Any]:
        e = self.e
        model_sd: dict[str, Any] = {}
        optim_state: dict[str, Any] = {}
        opt_of = {}
        if self.with_optim:
            opt_of[id(e.flat)] = e.optimizer
            if e.optimizer.partner is not None:
                opt_of[id(e.optimizer.partner.flat)] = e.optimizer.partner
        for name, f, off, shape, tp_dim in self._named_views(for_load=not write):
            so, sn = f.shard_offset, f.shard_numel
            if self.with_model:
                model_sd[name] = self._handle(f, off, shape, tp_dim, f.flat[so:so + sn], so, write)
            opt = opt_of.get(id(f))
            if opt is not None:
                st = {}
                for key in ("exp_avg", "exp_avg_sq", "master"):
                    buf = getattr(opt, key)
                    if buf.numel() == sn:  # SGD keeps no moments
                        st[key] = self._handle(f, off, shape, tp_dim, buf, so, write)
                optim_state[name] = st
        sd: dict[str, Any] = {"model": model_sd} if self.with_model else {}
        if self.with_model and hasattr(e.model, "_selection_biases"):
            # routers' selection biases: replicated buffers outside the flat buffers, named by global layer
            biases = dict(e.model._selection_biases(always=True))
            if biases:
                sd["buffers"] = biases
        if self.with_optim:
            sd["optim"] = {"state": optim_state, "meta": self._optim_meta()}
        rank = dist.get_rank() if dist.is_initialized() else 0
        rng = {f"rank{rank}": torch.get_rng_state()}
        if e.device.type == "cuda":
            rng[f"rank{rank}_cuda"] = torch.cuda.get_rng_state(e.device)
        sd["rng"] = rng
        return sd

    def _optim_meta(self) -> dict:
        o = self.e.optimizer
        return dict(step_count=o.step_count, sched_step=o.sched_step, kind=o.kind,
                    partner_step_count=o.partner.step_count if o.partner is not None else None)

    def state_dict(self) -> dict[str, Any]:
        write = self.available is None
        sd = self._build(write)
        if write:
            return sd
        # loading: request only what the checkpoint holds
        have = self.available
        pre = self.prefix

        def prune(d: dict, path: str) -> dict:
            out = {}
            for k, v in d.items():
                key = f"{path}{k}"
                if isinstance(v, dict) and not (key in have):
                    sub = prune(v, key + ".")
                    if sub:
                        out[k] = sub
                elif key in have:
                    out[k] = v
            return out

        pruned = prune(sd, pre)
        missing = [n for n in sd.get("model", {}) if n not in pruned.get("model", {})]
        if missing:
            raise KeyError(f"checkpoint has no tensor for {missing[:6]}{' ...' if len(missing) > 6 else ''}")
        return pruned

    def load_state_dict(self, sd: dict[str, Any]) -> None:
        """Runs after DCP filled the handles: publishes the loaded weight shards to every rank of the shard
        group, restores counters and generator state, and rebuilds whatever the checkpoint did not hold."""
        e = self.e
        for f in (e.flat, getattr(e, "flat_base", None), getattr(e, "flat_experts", None)):
            if f is None or not self.with_model:
                continue
            if f.dp_world > 1:
                so, sn = f.shard_offset, f.shard_numel
                mine = f.flat[so:so + sn].clone()
                if f.flat.is_cuda:
                    dist.all_gather_into_tensor(f.flat, mine, group=f.dp_group)
                else:
                    parts = [torch.empty_like(mine) for _ in range(f.dp_world)]
                    dist.all_gather(parts, mine, group=f.dp_group)
                    f.flat.copy_(torch.cat(parts))
        if e.optimizer is None:
            return
        opts = [e.optimizer] + ([e.optimizer.partner] if e.optimizer.partner is not None else [])
        osd = sd.get("optim") if self.with_optim else None
        for opt in opts:
            has_master = osd is not None and any("master" in st for st in osd.get("state", {}).values())
            if not has_master and not opt.host_state:
                opt.refresh_master()  # no master copy in the checkpoint: rebuild it from the loaded weights
        if osd is not None and isinstance(osd.get("meta"), dict):
            m = osd["meta"]
            self.loaded_optim_meta = m
            e.optimizer.step_count, e.optimizer.sched_step = int(m["step_count"]), int(m["sched_step"])
            if e.optimizer.partner is not None:
                e.optimizer.partner.sched_step = e.optimizer.sched_step
                pc = m.get("partner_step_count")
                e.optimizer.partner.step_count = int(pc if pc is not None else m["step_count"])
        rank = dist.get_rank() if dist.is_initialized() else 0
        rng = sd.get("rng", {})
        if f"rank{rank}" in rng:
            torch.set_rng_state(rng[f"rank{rank}"].cpu())
        if f"rank{rank}_cuda" in rng and e.device.type == "cuda":
            torch.cuda.set_rng_state(rng[f"rank{rank}_cuda"].cpu(), e.device)


def checkpoint_keys(path: str) -> set[str]:
    """Flattened keys of a DCP checkpoint directory (reads its ``.metadata`` only)."""
    from torch.distributed.checkpoint import FileSystemReader

    return set(FileSystemReader(path).read_metadata().state_dict_metadata.keys())


def _stage_to_host(obj: Any) -> Any:
    """Host copy of a state dict whose tensors are :class:`ShardedView` handles or plain tensors (pinned memory
    for device tensors, so the copies run asynchronously and one synchronise at the end suffices)."""
    if isinstance(obj, ShardedView):
        boxes = []
        for off, sz, t in obj._boxes:
            h = torch.empty(t.shape, dtype=t.dtype, pin_memory=t.is_cuda)
            h.copy_(t, non_blocking=True)
            boxes.append((off, sz, h))
        return ShardedView(tuple(obj.shape), obj.dtype, torch.device("cpu"), boxes)
    if torch.is_tensor(obj):
        h = torch.empty(obj.shape, dtype=obj.dtype, pin_memory=obj.is_cuda)
        h.copy_(obj, non_blocking=True)
        return h
    if isinstance(obj, dict):
        return {k: _stage_to_host(v) for k, v in obj.items()}
    return obj


def save_engine(engine, path: str, with_optim: bool = True, process_group=None, with_model: bool = True,
                executor=None):
    """``dcp.save`` of the engine state into ``path`` (collective over ``process_group``: every train rank).
    With ``executor`` (a one-thread pool) the state is first copied to pinned host memory, the call returns a
    future and the write runs on that thread; ``process_group`` must then be a gloo group that nothing else
    uses meanwhile (the counterpart of the staging in areal/utils/async_checkpoint.py:33-210)."""
    import torch.distributed.checkpoint as dcp

    st = EngineDCPState(engine, with_optim, with_model=with_model)
    kw: dict[str, Any] = dict(checkpoint_id=path)
    if dist.is_initialized():
        kw["process_group"] = process_group
    else:
        kw["no_dist"] = True
    if executor is None:
        dcp.save({"dcp": st}, **kw)
        return None
    staged = {"dcp": _stage_to_host(st.state_dict())}
    if engine.device.type == "cuda":
        torch.cuda.current_stream(engine.device).synchronize()
    return executor.submit(lambda: dcp.save(staged, **kw))


def load_engine(engine, path: str, with_optim: bool = True, process_group=None, with_model: bool = True):
    """``dcp.load`` into the engine, at any data-parallel size. Also reads the model part of a checkpoint
    written by the reference's FSDP engine (same names, fp32 tensors: they fill the weights and, when the
    checkpoint has no ``master`` entries, a second pass fills the fp32 master copy from the same tensors)."""
    import torch.distributed.checkpoint as dcp

    have = checkpoint_keys(path)
    st = EngineDCPState(engine, with_optim, available=have, with_model=with_model)
    kw: dict[str, Any] = dict(checkpoint_id=path)
    if dist.is_initialized():
        kw["process_group"] = process_group
    else:
        kw["no_dist"] = True
    dcp.load({"dcp": st}, **kw)
    opt = engine.optimizer
    if with_model and opt is not None and opt.kind != "adam_bf16" and not any(k.endswith(".master") for k in have):
        # fp32 weights stored under the model names (an FSDP2 checkpoint): they are the better master copy
        e = engine
        masters: dict[str, Any] = {}
        for name, f, off, shape, tp_dim in st._named_views(for_load=True):
            o = opt if f is e.flat else (opt.partner if opt.partner is not None and f is opt.partner.flat else None)
            if o is None or o.host_state:
                continue
            masters[name] = st._handle(f, off, shape, tp_dim, o.master, f.shard_offset, write=False)
        if masters:
            dcp.load({"dcp": {"model": masters}}, **kw)
    return st


def load_full_tensors(path: str, prefix: str = "dcp.model.") -> dict[str, torch.Tensor]:
    """Every tensor under ``prefix`` of a DCP checkpoint, assembled at full shape on this process (no process
    group): for conversion tools and tests."""
    import torch.distributed.checkpoint as dcp
    from torch.distributed.checkpoint import FileSystemReader
    from torch.distributed.checkpoint.metadata import TensorStorageMetadata

    md = FileSystemReader(path).read_metadata().state_dict_metadata
    want = {k: torch.empty(tuple(v.size), dtype=v.properties.dtype) for k, v in md.items()
            if k.startswith(prefix) and isinstance(v, TensorStorageMetadata)}
    dcp.load(want, checkpoint_id=path, no_dist=True)
    return {k[len(prefix):]: v for k, v in want.items()}
