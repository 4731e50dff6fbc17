"""Remote tensor handles.

In single-controller mode batches live on the workers; the controller only moves
*handles* (shape, dtype, owner address, shard id). ``remotize`` stores every
tensor of a nested structure in the local shard store and substitutes handles;
``localize`` turns handles back into tensors, fetching from the owner over HTTP
when it is another process (role of areal/infra/rpc/rtensor.py:392-447).

A handle may consist of several shards that live on different workers
(``RTensor.cat``: the rows of data-parallel ranks, concatenated along the first
dimension when the handle is localised, padded to the longest row length), so a
controller can "merge" the ranks' outputs without touching the data.

Transport is a backend (``get_backend`` / ``set_backend``): the default fetches
over the RPC servers' ``/data`` routes, all shards of one owner in one request;
``MemoryBackend`` serves tests and single-process runs. Fetched shards are kept
in a bounded buffer, since the same handle is typically localised by several
consumers (log-prob recomputation, advantage computation, the update).
"""

from __future__ import annotations

import io
import threading
import uuid
from dataclasses import dataclass
from typing import Any

import requests
import torch

from .serialization import deserialize_value, serialize_value


class ShardStore:
    """Per-process tensor store served at ``/data/<shard_id>`` by the RPC server."""

    def __init__(self):
        self._data: dict[str, torch.Tensor] = {}
        self._lock = threading.Lock()

    def put(self, shard_id: str, t: torch.Tensor):
        with self._lock:
            self._data[shard_id] = t

    def get(self, shard_id: str) -> torch.Tensor:
        with self._lock:
            return self._data[shard_id]

    def delete(self, shard_ids):
        with self._lock:
            for s in shard_ids:
                self._data.pop(s, None)

    def clear(self):
        with self._lock:
            n = len(self._data)
            self._data.clear()
            return n

    def __len__(self):
        return len(self._data)


LOCAL_STORE = ShardStore()
_LOCAL_ADDR: str | None = None


def set_local_addr(addr: str | None):
    global _LOCAL_ADDR
    _LOCAL_ADDR = addr


@dataclass
class TensorShardInfo:
    """One stored piece of a remote tensor: where it lives and how many rows it has."""
    shard_id: str
    addr: str | None  # "host:port" of the owning worker; None = this process
    rows: int = -1


class RTensorBackend:
    """Moves shards between processes. ``fetch`` gets several shards of ONE owner at once."""

    def store(self, addr: str, shard_id: str, t: torch.Tensor) -> None:
        raise NotImplementedError

    def fetch(self, addr: str, shard_ids: list[str], timeout: float = 600.0) -> list[torch.Tensor]:
        raise NotImplementedError

    def remove(self, addr: str, shard_ids: list[str]) -> None:
        raise NotImplementedError


class HttpRTensorBackend(RTensorBackend):
    """The RPC servers' ``/data`` routes (PUT one, POST ``/data/batch`` for many, POST ``/data/clear``)."""

    def store(self, addr, shard_id, t):
        r = requests.put(f"http://{addr}/data/{shard_id}", json=serialize_value(t.detach().cpu()), timeout=600)
        r.raise_for_status()

    def fetch(self, addr, shard_ids, timeout=600.0):
        if len(shard_ids) == 1:
            r = requests.get(f"http://{addr}/data/{shard_ids[0]}", timeout=timeout)
            r.raise_for_status()
            return [deserialize_value(r.json())]
        r = requests.post(f"http://{addr}/data/batch", json={"shard_ids": list(shard_ids)}, timeout=timeout)
        r.raise_for_status()
        return [deserialize_value(t) for t in r.json()["tensors"]]

    def remove(self, addr, shard_ids):
        requests.post(f"http://{addr}/data/clear", json={"shard_ids": list(shard_ids)}, timeout=60).raise_for_status()


class MemoryBackend(RTensorBackend):
    """Owners are entries of a dict of :class:`ShardStore` (tests; several logical workers in one process)."""

    def __init__(self):
        self.stores: dict[str, ShardStore] = {}
        self.fetches = 0

    def store(self, addr, shard_id, t):
        self.stores.setdefault(addr, ShardStore()).put(shard_id, t.detach().cpu())

    def fetch(self, addr, shard_ids, timeout=600.0):
        self.fetches += 1
        return [self.stores[addr].get(s) for s in shard_ids]

    def remove(self, addr, shard_ids):
        if addr in self.stores:
            self.stores[addr].delete(shard_ids)


class RayRTensorBackend(RTensorBackend):
    """Shards as objects of Ray's object store (``addr`` is ignored, the shard id is the hex of the object
    reference). Needs the ``ray`` package."""

    def __init__(self):
        try:
            import ray  # noqa: F401
        except ImportError as e:
            raise ImportError("RayRTensorBackend needs the `ray` package") from e
        self._refs: dict[str, Any] = {}

    def store(self, addr, shard_id, t):
        import ray

        self._refs[shard_id] = ray.put(t.detach().cpu())

    def fetch(self, addr, shard_ids, timeout=600.0):
        import ray

        return ray.get([self._refs[s] for s in shard_ids], timeout=timeout)

    def remove(self, addr, shard_ids):
        for s in shard_ids:
            self._refs.pop(s, None)


_BACKEND: RTensorBackend = HttpRTensorBackend()


def get_backend() -> RTensorBackend:
    return _BACKEND


def set_backend(backend: RTensorBackend | None) -> RTensorBackend:
    """Installs ``backend`` (``None``: the HTTP default); returns the previous one."""
    global _BACKEND
    prev, _BACKEND = _BACKEND, (backend or HttpRTensorBackend())
    return prev


# fetched shards, newest last; bounded by bytes
_FETCH_BUFFER: "dict[tuple[str, str], torch.Tensor]" = {}
_FETCH_LOCK = threading.Lock()
FETCH_BUFFER_BYTES = 1 << 30
_fetch_stats = {"hits": 0, "misses": 0, "requests": 0}


def _nbytes(t: torch.Tensor) -> int:
    return t.numel() * t.element_size()


def fetch(shards: list[TensorShardInfo], timeout: float = 600.0) -> list[torch.Tensor]:
    """The tensors of ``shards`` in order: local ones from the local store, remote ones from the fetch buffer or
    from their owner (one request per owner for everything that is missing)."""
    out: list[torch.Tensor | None] = [None] * len(shards)
    missing: dict[str, list[int]] = {}
    with _FETCH_LOCK:
        for i, sh in enumerate(shards):
            if sh.addr is None or sh.addr == _LOCAL_ADDR:
                out[i] = LOCAL_STORE.get(sh.shard_id)
            elif (sh.addr, sh.shard_id) in _FETCH_BUFFER:
                out[i] = _FETCH_BUFFER[(sh.addr, sh.shard_id)]
                _fetch_stats["hits"] += 1
            else:
                missing.setdefault(sh.addr, []).append(i)
                _fetch_stats["misses"] += 1
    for addr, idxs in missing.items():
        got = _BACKEND.fetch(addr, [shards[i].shard_id for i in idxs], timeout)
        with _FETCH_LOCK:
            _fetch_stats["requests"] += 1
            for i, t in zip(idxs, got):
                out[i] = t
                _FETCH_BUFFER[(addr, shards[i].shard_id)] = t
            total = sum(_nbytes(t) for t in _FETCH_BUFFER.values())
            while total > FETCH_BUFFER_BYTES and len(_FETCH_BUFFER) > 1:
                k = next(iter(_FETCH_BUFFER))
                total -= _nbytes(_FETCH_BUFFER.pop(k))
    return out  # type: ignore[return-value]


def store(t: torch.Tensor, addr: str | None = None, shard_id: str | None = None) -> TensorShardInfo:
    """Stores ``t`` here (``addr`` None or this process's address) or on another worker; returns its shard."""
    sid = shard_id or uuid.uuid4().hex
    if addr is None or addr == _LOCAL_ADDR:
        LOCAL_STORE.put(sid, t.detach().cpu())
        return TensorShardInfo(sid, _LOCAL_ADDR, t.shape[0] if t.dim() else -1)
    _BACKEND.store(addr, sid, t)
    return TensorShardInfo(sid, addr, t.shape[0] if t.dim() else -1)


def remove(shards: list[TensorShardInfo]) -> None:
    """Frees the shards at their owners and in the fetch buffer."""
    by_owner: dict[str | None, list[str]] = {}
    for sh in shards:
        by_owner.setdefault(sh.addr, []).append(sh.shard_id)
    for addr, ids in by_owner.items():
        if addr is None or addr == _LOCAL_ADDR:
            LOCAL_STORE.delete(ids)
        else:
            _BACKEND.remove(addr, ids)
    with _FETCH_LOCK:
        for sh in shards:
            _FETCH_BUFFER.pop((sh.addr, sh.shard_id), None)


def clear_fetch_buffer() -> int:
    with _FETCH_LOCK:
        n = len(_FETCH_BUFFER)
        _FETCH_BUFFER.clear()
        return n


def fetch_buffer_stats() -> dict[str, int]:
    with _FETCH_LOCK:
        return dict(_fetch_stats, entries=len(_FETCH_BUFFER), bytes=sum(_nbytes(t) for t in _FETCH_BUFFER.values()))


def storage_stats() -> dict[str, int]:
    """What this process's shard store holds."""
    with LOCAL_STORE._lock:
        return {"entries": len(LOCAL_STORE._data), "bytes": sum(_nbytes(t) for t in LOCAL_STORE._data.values())}


def flatten_shard_ids(obj: Any) -> list[str]:
    return [sid for _, sid in collect_shard_ids(obj)]


@dataclass
class RTensor:
    shard_id: str
    addr: str | None  # "host:port" of the owning worker; None = this process
    shape: tuple
    dtype: str
    shards: list | None = None  # several pieces, concatenated along dim 0 (``shard_id`` / ``addr`` are the first's)

    def __rtensor__(self) -> dict:
        d = {"__type__": "rtensor", "shard_id": self.shard_id, "addr": self.addr, "shape": list(self.shape),
             "dtype": self.dtype}
        if self.shards:
            d["shards"] = [[s.shard_id, s.addr, s.rows] for s in self.shards]
        return d

    @classmethod
    def from_dict(cls, d: dict) -> "RTensor":
        shards = [TensorShardInfo(*s) for s in d["shards"]] if d.get("shards") else None
        return cls(d["shard_id"], d["addr"], tuple(d["shape"]), d["dtype"], shards)

    @property
    def meta(self) -> torch.Tensor:
        return torch.empty(self.shape, dtype=getattr(torch, self.dtype), device="meta")

    def shard_infos(self) -> list[TensorShardInfo]:
        return list(self.shards) if self.shards else [TensorShardInfo(self.shard_id, self.addr, self.shape[0] if self.shape else -1)]

    @classmethod
    def cat(cls, parts: "list[RTensor]") -> "RTensor":
        """One handle over the rows of ``parts`` (first dimensions add up; a second, sequence dimension is padded
        to the longest when the handle is localised). No data moves."""
        if not parts:
            raise ValueError("nothing to concatenate")
        if len({p.dtype for p in parts}) != 1 or len({len(p.shape) for p in parts}) != 1:
            raise ValueError("parts differ in dtype or rank")
        infos = [s for p in parts for s in p.shard_infos()]
        rows = sum(p.shape[0] for p in parts)
        rest = tuple(max(p.shape[i] for p in parts) for i in range(1, len(parts[0].shape)))
        return cls(infos[0].shard_id, infos[0].addr, (rows,) + rest, parts[0].dtype, infos)

    def to_local(self, timeout: float = 600.0) -> torch.Tensor:
        pieces = fetch(self.shard_infos(), timeout)
        if len(pieces) == 1:
            return pieces[0]
        if pieces[0].dim() >= 2 and len({p.shape[1] for p in pieces}) > 1:
            L = max(p.shape[1] for p in pieces)
            pieces = [torch.nn.functional.pad(p, [0, 0] * (p.dim() - 2) + [0, L - p.shape[1]]) for p in pieces]
        return torch.cat(pieces, 0)


def remotize(obj: Any, store: ShardStore | None = None, addr: str | None = None) -> Any:
    store = store or LOCAL_STORE
    addr = addr if addr is not None else _LOCAL_ADDR
    if torch.is_tensor(obj):
        sid = uuid.uuid4().hex
        store.put(sid, obj.detach().cpu())
        return RTensor(sid, addr, tuple(obj.shape), str(obj.dtype).replace("torch.", ""))
    if isinstance(obj, dict):
        return {k: remotize(v, store, addr) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return type(obj)(remotize(v, store, addr) for v in obj)
    return obj


def localize(obj: Any) -> Any:
    if isinstance(obj, RTensor):
        return obj.to_local()
    if isinstance(obj, dict):
        return {k: localize(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return type(obj)(localize(v) for v in obj)
    return obj


def collect_shard_ids(obj: Any) -> list[tuple[str | None, str]]:
    out = []
    if isinstance(obj, RTensor):
        out += [(s.addr, s.shard_id) for s in obj.shard_infos()]
    elif isinstance(obj, dict):
        for v in obj.values():
            out += collect_shard_ids(v)
    elif isinstance(obj, (list, tuple)):
        for v in obj:
            out += collect_shard_ids(v)
    return out
