"""Distributed statistics tracker.

Two usage styles (areal/utils/stats_tracker.py:31-332 in the reference):

* batched, masked tensors in train engines: ``denominator(n_tokens=mask)`` then
  ``stat(loss=tensor, denominator="n_tokens")`` – exported as masked
  mean/min/max over all ranks;
* streaming scalars in rollout workers: ``scalar(reward=1.0)`` – exported as
  means with a ``__count`` companion so a controller can merge workers.

``export`` synchronises the key set across ranks (``all_gather_object``) and
reduces values with ``all_reduce``.
"""

from __future__ import annotations

import time
from collections import defaultdict
from contextlib import contextmanager
from enum import Enum, auto
from typing import Any

import torch
import torch.distributed as dist


class ReduceType(Enum):
    AVG_MIN_MAX = auto()
    AVG = auto()
    SUM = auto()
    MIN = auto()
    MAX = auto()
    SCALAR = auto()


class DistributedStatsTracker:
    def __init__(self, name: str = ""):
        self.name = name
        self._scope: list[str] = [name] if name else []
        self._denoms: dict[str, list[torch.Tensor]] = defaultdict(list)
        self._stats: dict[str, list[torch.Tensor]] = defaultdict(list)
        self._denom_of: dict[str, str] = {}
        self._reduce: dict[str, ReduceType] = {}
        self._scalars: dict[str, list[float]] = defaultdict(list)

    # ------------------------------------------------------------- scoping
    @contextmanager
    def scope(self, name: str):
        self._scope.append(name.strip("/"))
        try:
            yield
        finally:
            self._scope.pop()

    def _key(self, k: str) -> str:
        return "/".join(self._scope + [k]) if self._scope else k

    @contextmanager
    def record_timing(self, key: str):
        from . import perf_tracer  # every timed phase is also a scope of the perf trace (when one is configured)

        t0 = time.perf_counter()
        try:
            with perf_tracer.trace_scope(key, perf_tracer.Category.COMPUTE):
                yield
        finally:
            self._scalars["/".join(["timeperf", key])].append(time.perf_counter() - t0)
            self._reduce.setdefault("timeperf/" + key, ReduceType.SCALAR)

    # ------------------------------------------------------------ recording
    def denominator(self, **kwargs: torch.Tensor):
        for k, v in kwargs.items():
            if v.dtype != torch.bool:
                raise ValueError(f"denominator {k} must be a bool tensor")
            key = self._key(k)
            self._denoms[key].append(v.detach().reshape(-1).clone())
            self._reduce[key] = ReduceType.SUM

    def stat(self, denominator: str, reduce_type: ReduceType | None = None, **kwargs: torch.Tensor):
        dkey = self._key(denominator)
        if dkey not in self._denoms:
            raise ValueError(f"denominator {denominator} has not been recorded")
        for k, v in kwargs.items():
            key = self._key(k)
            d = self._denoms[dkey][-1]
            v = v.detach().float().reshape(-1)
            if v.shape != d.shape:
                raise ValueError(f"stat {k} has shape {tuple(v.shape)}, denominator {tuple(d.shape)}")
            self._stats[key].append(v)
            self._denom_of[key] = dkey
            self._reduce[key] = reduce_type or ReduceType.AVG_MIN_MAX

    def scalar(self, **kwargs: float):
        for k, v in kwargs.items():
            key = self._key(k)
            self._scalars[key].append(float(v))
            self._reduce[key] = ReduceType.SCALAR

    # -------------------------------------------------------------- export
    def export(self, key: str | None = None, reduce_group=None, reset: bool = True) -> dict[str, float]:
        distributed = dist.is_initialized() and (reduce_group is not None or dist.get_world_size() > 1)
        keys = sorted(set(self._stats) | set(self._denoms) | set(self._scalars))
        if key is not None:
            keys = [k for k in keys if k == key or k.startswith(key.rstrip("/") + "/")]
        types = {k: self._reduce[k].name for k in keys}
        if distributed:
            gathered: list[Any] = [None] * dist.get_world_size(reduce_group)
            dist.all_gather_object(gathered, types, group=reduce_group)
            merged: dict[str, str] = {}
            for g in gathered:
                merged.update(g)
            types = merged
            keys = sorted(types)
        dev = self._device(reduce_group)
        out: dict[str, float] = {}

        def reduce(t: torch.Tensor, op):
            t = t.to(dev)
            if distributed:
                dist.all_reduce(t, op=op, group=reduce_group)
            return t

        for k in keys:
            rt = ReduceType[types[k]]
            if rt == ReduceType.SCALAR:
                vals = self._scalars.get(k, [])
                buf = reduce(torch.tensor([sum(vals), float(len(vals))], dtype=torch.float64), dist.ReduceOp.SUM)
                if float(buf[1]) > 0:
                    out[k] = float(buf[0] / buf[1])
                    out[k + "__count"] = float(buf[1])
                continue
            if k in self._denoms or (k not in self._stats and k not in self._denom_of):
                n = sum(int(d.sum()) for d in self._denoms.get(k, []))
                out[k] = float(reduce(torch.tensor([float(n)], dtype=torch.float64), dist.ReduceOp.SUM)[0])
                continue
            dk = self._denom_of.get(k)
            vs = self._stats.get(k, [])
            ds = self._denoms.get(dk, [])[-len(vs):] if vs else []
            # pair each stat with the denominator recorded at the same time
            pairs = list(zip(vs, self._pair_denoms(k)))
            s = sum((float((v * d.to(v.device)).sum()) for v, d in pairs), 0.0)
            n = sum((float(d.sum()) for _, d in pairs), 0.0)
            mn = min((float(v[d.to(v.device)].min()) for v, d in pairs if bool(d.any())), default=float("inf"))
            mx = max((float(v[d.to(v.device)].max()) for v, d in pairs if bool(d.any())), default=float("-inf"))
            tot = reduce(torch.tensor([s, n], dtype=torch.float64), dist.ReduceOp.SUM)
            if rt in (ReduceType.AVG_MIN_MAX, ReduceType.AVG):
                if float(tot[1]) == 0:
                    continue
                avg = float(tot[0] / tot[1])
                if rt == ReduceType.AVG:
                    out[k] = avg
                else:
                    out[k + "/avg"] = avg
                    out[k + "/min"] = float(reduce(torch.tensor([mn], dtype=torch.float64), dist.ReduceOp.MIN)[0])
                    out[k + "/max"] = float(reduce(torch.tensor([mx], dtype=torch.float64), dist.ReduceOp.MAX)[0])
            elif rt == ReduceType.SUM:
                out[k] = float(tot[0])
            elif rt == ReduceType.MIN:
                out[k] = float(reduce(torch.tensor([mn], dtype=torch.float64), dist.ReduceOp.MIN)[0])
            elif rt == ReduceType.MAX:
                out[k] = float(reduce(torch.tensor([mx], dtype=torch.float64), dist.ReduceOp.MAX)[0])
        if reset:
            self._reset(keys if key is not None else None)
        return out

    def _pair_denoms(self, stat_key: str) -> list[torch.Tensor]:
        dk = self._denom_of[stat_key]
        n = len(self._stats[stat_key])
        ds = self._denoms[dk]
        shapes = [v.shape for v in self._stats[stat_key]]
        # match from the end: stats are recorded right after their denominators
        out, j = [], len(ds) - 1
        for sh in reversed(shapes):
            while j >= 0 and ds[j].shape != sh:
                j -= 1
            out.append(ds[max(j, 0)])
            j -= 1
        return out[::-1]

    def _device(self, group):
        if dist.is_initialized() and dist.get_backend(group) == "nccl":
            return torch.device("cuda", torch.cuda.current_device())
        return torch.device("cpu")

    def _reset(self, keys=None):
        if keys is None:
            self._denoms.clear(); self._stats.clear(); self._scalars.clear()
            self._denom_of.clear(); self._reduce.clear()
            return
        for k in keys:
            self._denoms.pop(k, None); self._stats.pop(k, None); self._scalars.pop(k, None)
            self._denom_of.pop(k, None); self._reduce.pop(k, None)


DEFAULT_TRACKER = DistributedStatsTracker()
_TRACKERS: dict[str, DistributedStatsTracker] = {}

stat = DEFAULT_TRACKER.stat
denominator = DEFAULT_TRACKER.denominator
scalar = DEFAULT_TRACKER.scalar
scope = DEFAULT_TRACKER.scope
record_timing = DEFAULT_TRACKER.record_timing
export = DEFAULT_TRACKER.export


def get(name: str = "") -> DistributedStatsTracker:
    if not name:
        return DEFAULT_TRACKER
    if name not in _TRACKERS:
        _TRACKERS[name] = DistributedStatsTracker(name)
    return _TRACKERS[name]


def export_all(reduce_group=None, reset: bool = True) -> dict[str, float]:
    out = DEFAULT_TRACKER.export(reduce_group=reduce_group, reset=reset)
    if dist.is_initialized():
        names: list[Any] = [None] * dist.get_world_size(reduce_group)
        dist.all_gather_object(names, sorted(_TRACKERS), group=reduce_group)
        all_names = sorted({n for ns in names for n in ns})
    else:
        all_names = sorted(_TRACKERS)
    for n in all_names:
        out.update(get(n).export(reduce_group=reduce_group, reset=reset))
    return out


def merge_scalar_stats(stats_list: list[dict[str, float]]) -> dict[str, float]:
    """Merges exports of several workers using their ``__count`` weights."""
    sums: dict[str, float] = defaultdict(float)
    counts: dict[str, float] = defaultdict(float)
    plain: dict[str, list[float]] = defaultdict(list)
    for st in stats_list:
        for k, v in st.items():
            if k.endswith("__count"):
                continue
            c = st.get(k + "__count")
            if c is None:
                plain[k].append(v)
            else:
                sums[k] += v * c
                counts[k] += c
    out = {k: sums[k] / counts[k] for k in sums if counts[k] > 0}
    out.update({k + "__count": counts[k] for k in counts})
    out.update({k: sum(v) / len(v) for k, v in plain.items()})
    return out
