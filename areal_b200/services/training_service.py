"""Training service: a gateway that owns a set of train-engine workers (one per data-parallel
rank), splits every incoming batch across them (token-balanced, groups kept together), calls the
same engine method on all of them concurrently and merges the results.
Reference: areal/experimental/training_service/{gateway,router,data_proxy/dispatcher,worker}."""

from __future__ import annotations

from concurrent.futures import ThreadPoolExecutor
from typing import Any

from fastapi import FastAPI, HTTPException, Request

from ..infra.controller.train_controller import dispatch_batch, merge_outputs
from ..infra.rpc.serialization import deserialize_value, serialize_value
from ..infra.utils.http import request_with_retry
from .base import WorkerRegistry, make_auth


def create_gateway_app(token: str | None = None, post=None) -> FastAPI:
    app = FastAPI()
    reg = WorkerRegistry("round_robin")
    auth = make_auth(token)
    post = post or (lambda url, body: request_with_retry("POST", url, json=body, max_retries=0, timeout=7200).json())
    pool = ThreadPoolExecutor(max_workers=64, thread_name_prefix="train-gw")

    def ranks() -> list[dict]:
        ws = sorted(reg.snapshot(), key=lambda w: w.get("rank", 0))
        if not ws:
            raise HTTPException(status_code=503, detail="no train worker is registered")
        return ws

    def call_all(method: str, per_rank_args: list[list[Any]], kwargs: dict) -> list[Any]:
        ws = ranks()

        def one(i):
            body = {"method": method, "args": serialize_value(per_rank_args[i]), "kwargs": serialize_value(kwargs)}
            return deserialize_value(post(f"http://{ws[i]['addr']}/call", body)["result"])

        return list(pool.map(one, range(len(ws))))

    @app.post("/register")
    async def register(req: Request):
        auth(req)
        b = await req.json()
        reg.register(b["worker_id"], b["addr"], rank=int(b.get("rank", len(reg.snapshot()))))
        return {"workers": len(reg.snapshot())}

    @app.post("/call")
    async def call(req: Request):
        """``{"method", "batch"?, "args", "kwargs", "group_size"?}``: with ``batch`` the tensor dict is
        split across ranks and passed as first argument; without it every rank gets the same call."""
        auth(req)
        b = await req.json()
        args = deserialize_value(b.get("args", []))
        kwargs = deserialize_value(b.get("kwargs", {}))
        n = len(ranks())
        if b.get("batch") is not None:
            batch = deserialize_value(b["batch"])
            shards, order = dispatch_batch(batch, n, group_size=int(b.get("group_size", 1)))
            outs = call_all(b["method"], [[s, *args] for s in shards], kwargs)
            return {"result": serialize_value(merge_outputs(outs, order))}
        outs = call_all(b["method"], [list(args)] * n, kwargs)
        return {"result": serialize_value(outs[0] if all(o == outs[0] for o in outs[1:]) else outs)}

    app.state.registry = reg
    return app
