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

    @app.post("/workers")
    async def workers(req: Request):
        auth(req)
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


class GatewayTrainEngine:
    """The script's handle on a training service: the ``TrainEngine`` calls a trainer makes, carried out through
    the gateway's ``/call`` route (which splits batches over the data-parallel workers by tokens and merges the
    per-sample results). Data methods take a padded batch; evaluation and inference batches that do not divide
    over the workers are topped up with weightless samples and trimmed again. Loss functions travel by import
    path (``"pkg.module.fn"``), since the workers are other processes.
    Reference: areal/experimental/training_service/controller/controller.py (GatewayTrainController)."""

    def __init__(self, gateway_url: str, token: str | None = None, group_size: int = 1, post=None):
        self.url, self.token, self.group_size = gateway_url.rstrip("/"), token, group_size
        self._post = post or (lambda url, body, headers: request_with_retry(
            "POST", url, json=body, headers=headers, max_retries=0, timeout=7200).json())
        self._version = 0

    def _headers(self) -> dict[str, str]:
        return {"Authorization": f"Bearer {self.token}"} if self.token else {}

    def _call(self, method: str, *args, batch: dict | None = None, **kwargs):
        body = {"method": method, "args": serialize_value(list(args)), "kwargs": serialize_value(kwargs),
                "group_size": self.group_size}
        if batch is not None:
            body["batch"] = serialize_value(batch)
        return deserialize_value(self._post(self.url + "/call", body, self._headers())["result"])

    def n_workers(self) -> int:
        return int(self._post(self.url + "/workers", {}, self._headers())["workers"])

    @staticmethod
    def _fn_path(fn) -> str:
        if isinstance(fn, str):
            return fn
        path = f"{fn.__module__}.{fn.__qualname__}"
        if "<locals>" in path or "<lambda>" in path:
            raise ValueError("functions sent to a training service must be importable (module-level): "
                             f"got {path}")
        return path

    # ------------------------------------------------------------------ data methods
    def train_batch(self, input_: dict, loss_fn, loss_weight_fn):
        return self._call("train_batch", self._fn_path(loss_fn), self._fn_path(loss_weight_fn), batch=input_)

    def _padded(self, method: str, input_: dict, *args, **kwargs):
        from ..infra.controller.train_controller import pad_batch_for_dispatch, strip_padding

        n_real = input_["attention_mask"].shape[0]
        batch, n_pad = pad_batch_for_dispatch(input_, self.n_workers(), self.group_size)
        return strip_padding(self._call(method, *args, batch=batch, **kwargs), n_real, n_pad)

    def eval_batch(self, input_: dict, loss_fn, loss_weight_fn):
        return self._padded("eval_batch", input_, self._fn_path(loss_fn), self._fn_path(loss_weight_fn))

    def forward_batch(self, input_: dict, **kwargs):
        return self._padded("forward_batch", input_, **kwargs)

    # ------------------------------------------------------------------ control
    def set_version(self, version: int):
        self._version = int(version)
        self._call("set_version", int(version))

    def get_version(self) -> int:
        return self._version

    def train(self, mode: bool = True):
        self._call("train", mode)
        return self

    def eval(self):
        return self.train(False)

    def step_lr_scheduler(self):
        self._call("step_lr_scheduler")

    def save(self, meta):
        self._call("save", meta)

    def load(self, meta):
        self._call("load", meta)

    def update_weights(self, meta):
        self._call("update_weights", meta)

    def export_stats(self) -> dict:
        out = self._call("export_stats")
        return out[0] if isinstance(out, list) else out
