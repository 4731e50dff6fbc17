"""Weight-update service: the rendezvous between training and inference for weight transfers.

Training and inference sides ``/connect`` with their role, rank and how their copy of the weights
can be reached (a disk path, or the CUDA IPC handles of a rollout engine's flat buffer for the
NVLink peer-to-peer path); the gateway pairs trainers with rollout engines, keeps a small KV of
weight metadata per version (``/weight_meta/{key}``) and sequences an ``/update_weights`` round:
pause inference → tell the trainers to push (or the engines to load from disk) → bump the
version → resume. Transfers themselves never pass through the service.
Reference: areal/experimental/weight_update/{gateway/app.py:194-799,controller}.
"""

from __future__ import annotations

import threading
import time
from typing import Any

from fastapi import FastAPI, HTTPException, Request

from ..infra.rpc.serialization import deserialize_value, serialize_value
from ..infra.utils.http import request_with_retry
from .base import make_auth


def pair_ranks(n_train: int, n_infer: int) -> dict[int, list[int]]:
    """Which inference engines each trainer rank feeds: engines are dealt round-robin, so every
    engine has exactly one source and the load differs by at most one."""
    out: dict[int, list[int]] = {r: [] for r in range(n_train)}
    for e in range(n_infer):
        out[e % n_train].append(e)
    return out


def create_gateway_app(token: str | None = None, post=None) -> FastAPI:
    app = FastAPI()
    auth = make_auth(token)
    post = post or (lambda url, body: request_with_retry("POST", url, json=body, max_retries=0, timeout=3600).json())
    members: dict[str, dict[int, dict]] = {"train": {}, "inference": {}}
    kv: dict[str, Any] = {}
    state = {"version": 0, "updating": False, "history": []}
    lock = threading.Lock()

    def call(addr: str, method: str, *args, **kwargs):
        body = {"method": method, "args": serialize_value(list(args)), "kwargs": serialize_value(kwargs)}
        return deserialize_value(post(f"http://{addr}/call", body)["result"])

    @app.post("/connect")
    async def connect(req: Request):
        auth(req)
        b = await req.json()
        role = b["role"]
        if role not in members:
            raise HTTPException(status_code=400, detail="role must be 'train' or 'inference'")
        members[role][int(b["rank"])] = {"addr": b["addr"], "info": deserialize_value(b.get("info"))}
        return {"role": role, "rank": int(b["rank"]), "train": len(members["train"]), "inference": len(members["inference"]),
                "version": state["version"]}

    @app.post("/disconnect")
    async def disconnect(req: Request):
        auth(req)
        b = await req.json()
        members.get(b["role"], {}).pop(int(b["rank"]), None)
        return {"train": len(members["train"]), "inference": len(members["inference"])}

    @app.get("/plan")
    def plan(req: Request):
        auth(req)
        return {"pairs": pair_ranks(max(len(members["train"]), 1), len(members["inference"])),
                "inference": {r: m["info"] for r, m in members["inference"].items()}}

    @app.put("/weight_meta/{key:path}")
    async def put_meta(key: str, req: Request):
        auth(req)
        kv[key] = await req.json()
        return {"key": key}

    @app.get("/weight_meta/{key:path}")
    def get_meta(key: str, req: Request):
        auth(req)
        if key not in kv:
            raise HTTPException(status_code=404, detail=f"no weight metadata under {key!r}")
        return kv[key]

    @app.delete("/weight_meta/{key:path}")
    def del_meta(key: str, req: Request):
        auth(req)
        return {"deleted": kv.pop(key, None) is not None}

    @app.post("/update_weights")
    async def update(req: Request):
        auth(req)
        b = await req.json()
        meta = deserialize_value(b.get("meta"))
        if not members["inference"]:
            raise HTTPException(status_code=409, detail="no inference engine is connected")
        with lock:
            if state["updating"]:
                raise HTTPException(status_code=409, detail="a weight update is already running")
            state["updating"] = True
        t0 = time.perf_counter()
        try:
            version = int(b.get("version", state["version"] + 1))
            engines = [m["addr"] for _, m in sorted(members["inference"].items())]
            for a in engines:
                call(a, "pause_generation")
            if b.get("mode", "disk") == "disk":
                for a in engines:
                    call(a, "update_weights_from_disk", meta)
            else:  # trainers push into the engines' buffers themselves
                for _, m in sorted(members["train"].items()):
                    call(m["addr"], "update_weights", meta)
            for a in engines:
                call(a, "set_version", version)
                call(a, "continue_generation")
            state["version"] = version
            dt = time.perf_counter() - t0
            state["history"].append({"version": version, "seconds": dt})
            return {"version": version, "seconds": dt}
        finally:
            state["updating"] = False

    @app.get("/status")
    def status(req: Request):
        auth(req)
        return {"version": state["version"], "updating": state["updating"], "history": state["history"][-20:],
                "train": sorted(members["train"]), "inference": sorted(members["inference"])}

    return app
