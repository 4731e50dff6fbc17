"""Remote tensor handles.

In single-controller mode batches live on the workers; the controller only moves
*handles* (shape, dtype, owner address, shard id). ``remotize`` stores every
tensor of a nested structure in the local shard store and substitutes handles;
``localize`` turns handles back into tensors, fetching from the owner over HTTP
when it is another process (role of areal/infra/rpc/rtensor.py:392-447).
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
class RTensor:
    shard_id: str
    addr: str | None  # "host:port" of the owning worker; None = this process
    shape: tuple
    dtype: str

    def __rtensor__(self) -> dict:
        return {"__type__": "rtensor", "shard_id": self.shard_id, "addr": self.addr, "shape": list(self.shape),
                "dtype": self.dtype}

    @classmethod
    def from_dict(cls, d: dict) -> "RTensor":
        return cls(d["shard_id"], d["addr"], tuple(d["shape"]), d["dtype"])

    @property
    def meta(self) -> torch.Tensor:
        return torch.empty(self.shape, dtype=getattr(torch, self.dtype), device="meta")

    def to_local(self, timeout: float = 600.0) -> torch.Tensor:
        if self.addr is None or self.addr == _LOCAL_ADDR:
            return LOCAL_STORE.get(self.shard_id)
        r = requests.get(f"http://{self.addr}/data/{self.shard_id}", timeout=timeout)
        r.raise_for_status()
        return deserialize_value(r.json())


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
        out.append((obj.addr, obj.shard_id))
    elif isinstance(obj, dict):
        for v in obj.values():
            out += collect_shard_ids(v)
    elif isinstance(obj, (list, tuple)):
        for v in obj:
            out += collect_shard_ids(v)
    return out
