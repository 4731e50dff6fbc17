"""Remote dataset service: dataset shards live in worker processes; trainers pull batches by
index through ``RDataset`` so that tokenisation / decoding cost stays off the training hosts.

* worker app  – ``/load`` a dataset (registry name or import path + kwargs), ``/len``, ``/fetch``
                indices, ``/health``;
* router/gateway app – registers workers, shards datasets across them by index (``i % n``),
                fans ``/fetch`` out and merges in request order;
* ``RDataset`` – map-style dataset over the gateway; ``PrefetchingSampler`` keeps the next
                batches' fetches in flight.
Reference: areal/infra/data_service/{controller,gateway,router,worker}, rdataset.py.
"""

from __future__ import annotations

import importlib
import threading
from collections import deque
from concurrent.futures import Future, ThreadPoolExecutor
from typing import Any, Iterator

from fastapi import FastAPI, HTTPException, Request

from ..infra.rpc.serialization import deserialize_value, serialize_value
from ..infra.utils.http import request_with_retry
from .base import WorkerRegistry, make_auth


def create_worker_app() -> FastAPI:
    app = FastAPI()
    datasets: dict[str, Any] = {}

    @app.get("/health")
    def health():
        return {"status": "ok", "datasets": sorted(datasets)}

    @app.post("/load")
    async def load(req: Request):
        body = await req.json()
        name, spec, kwargs = body["name"], body["dataset"], deserialize_value(body.get("kwargs", {}))
        ds = None
        if "." in spec and "/" not in spec:  # "package.module.factory"
            mod, _, attr = spec.rpartition(".")
            try:
                ds = getattr(importlib.import_module(mod), attr)(**kwargs)
            except (ImportError, AttributeError):
                ds = None
        if ds is None:  # a dataset path / name known to the dataset registry
            from ..dataset import get_custom_dataset

            ds = get_custom_dataset(path=spec, **kwargs)
        datasets[name] = ds
        return {"name": name, "len": len(ds)}

    @app.post("/len")
    async def length(req: Request):
        name = (await req.json())["name"]
        if name not in datasets:
            raise HTTPException(status_code=404, detail=f"dataset {name!r} is not loaded")
        return {"len": len(datasets[name])}

    @app.post("/fetch")
    async def fetch(req: Request):
        body = await req.json()
        ds = datasets.get(body["name"])
        if ds is None:
            raise HTTPException(status_code=404, detail=f"dataset {body['name']!r} is not loaded")
        return {"items": serialize_value([ds[i] for i in body["indices"]])}

    app.state.datasets = datasets
    return app


def create_gateway_app(token: str | None = None, post=None) -> FastAPI:
    """``post(url, json) -> dict`` is injectable (tests route it to in-process worker apps)."""
    app = FastAPI()
    reg = WorkerRegistry("round_robin")
    auth = make_auth(token)
    post = post or (lambda url, body: request_with_retry("POST", url, json=body).json())
    lengths: dict[str, int] = {}

    def workers():
        ws = [w for w in reg.snapshot() if w["healthy"]]
        if not ws:
            raise HTTPException(status_code=503, detail="no data worker is registered")
        return ws

    @app.post("/register")
    async def register(req: Request):
        auth(req)
        b = await req.json()
        reg.register(b["worker_id"], b["addr"])
        return {"workers": len(reg.snapshot())}

    @app.post("/load")
    async def load(req: Request):
        auth(req)
        body = await req.json()
        n = None
        for w in workers():  # every worker loads the dataset; indices are sharded at fetch time
            n = post(f"http://{w['addr']}/load", body)["len"]
        lengths[body["name"]] = n
        return {"name": body["name"], "len": n}

    @app.post("/len")
    async def length(req: Request):
        auth(req)
        name = (await req.json())["name"]
        if name not in lengths:
            raise HTTPException(status_code=404, detail=f"dataset {name!r} is not loaded")
        return {"len": lengths[name]}

    @app.post("/fetch")
    async def fetch(req: Request):
        auth(req)
        body = await req.json()
        ws = workers()
        idx = list(body["indices"])
        buckets: dict[int, list[int]] = {}
        for pos, i in enumerate(idx):
            buckets.setdefault(i % len(ws), []).append(pos)
        out: list[Any] = [None] * len(idx)
        for wi, positions in buckets.items():
            r = post(f"http://{ws[wi]['addr']}/fetch", {"name": body["name"], "indices": [idx[p] for p in positions]})
            for p, item in zip(positions, deserialize_value(r["items"])):
                out[p] = item
        return {"items": serialize_value(out)}

    app.state.registry = reg
    return app


class RDataset:
    """Map-style dataset whose items come from the data service."""

    def __init__(self, gateway_addr: str, name: str, token: str | None = None, post=None):
        self.addr = gateway_addr if gateway_addr.startswith("http") else "http://" + gateway_addr
        self.name, self.token = name, token
        self._post = post or self._http_post
        self._len: int | None = None

    def _http_post(self, path: str, body: dict) -> dict:
        import requests

        headers = {"Authorization": f"Bearer {self.token}"} if self.token else {}
        r = requests.post(self.addr + path, json=body, headers=headers, timeout=300)
        r.raise_for_status()
        return r.json()

    def __len__(self) -> int:
        if self._len is None:
            self._len = int(self._post("/len", {"name": self.name})["len"])
        return self._len

    def fetch(self, indices: list[int]) -> list[Any]:
        return deserialize_value(self._post("/fetch", {"name": self.name, "indices": list(indices)})["items"])

    def __getitem__(self, i: int) -> Any:
        return self.fetch([i])[0]


class PrefetchingSampler:
    """Iterates ``batches`` (lists of indices) over an :class:`RDataset` with ``depth`` fetches
    in flight ahead of the consumer."""

    def __init__(self, dataset: RDataset, batches: list[list[int]], depth: int = 2):
        self.dataset, self.batches, self.depth = dataset, batches, max(1, depth)
        self._pool = ThreadPoolExecutor(max_workers=self.depth, thread_name_prefix="rdata")
        self._lock = threading.Lock()

    def __len__(self):
        return len(self.batches)

    def __iter__(self) -> Iterator[list[Any]]:
        pending: deque[Future] = deque()
        it = iter(self.batches)
        for _ in range(self.depth):
            b = next(it, None)
            if b is not None:
                pending.append(self._pool.submit(self.dataset.fetch, b))
        while pending:
            items = pending.popleft().result()
            b = next(it, None)
            if b is not None:
                pending.append(self._pool.submit(self.dataset.fetch, b))
            yield items
