"""Worker-side RPC server for single-controller mode.

    python -m areal_b200.infra.rpc.rpc_server --port 0 [--host 127.0.0.1] [--name-key KEY]

Endpoints (FastAPI / uvicorn): ``/health``, ``/alloc_ports``, ``/set_env``,
``/configure``, ``/create_engine``, ``/call``, ``/data/<shard_id>`` (PUT / GET),
``/data/batch``, ``/data/clear``, ``/fork``, ``/kill_forked_worker``. All engine
work (creation and method calls) runs on ONE dedicated engine thread, so
collective calls issued by different requests can never interleave. Arguments
and results cross the wire in the envelopes of ``serialization.py``; tensors may
travel as ``RTensor`` handles that are resolved worker-side.

This is the counterpart of the reference's Flask "guard" application and engine
blueprint (areal/infra/rpc/guard/app.py, engine_blueprint.py:114-605,
data_blueprint.py).
"""

from __future__ import annotations

import argparse
import importlib
import os
import queue
import signal
import socket
import subprocess
import sys
import threading
import traceback
from concurrent.futures import Future
from typing import Any

import uvicorn
from fastapi import FastAPI, HTTPException, Request

from ...utils import logging, perf_tracer
from . import rtensor
from .serialization import deserialize_value, serialize_value

logger = logging.getLogger("RPCServer")


class EngineThread:
    """Serialises every engine operation of this worker on one thread."""

    def __init__(self):
        self._q: queue.Queue = queue.Queue()
        self._t = threading.Thread(target=self._run, name="engine-thread", daemon=True)
        self._t.start()

    def _run(self):
        while True:
            fn, fut = self._q.get()
            if fn is None:
                return
            try:
                fut.set_result(fn())
            except BaseException as e:
                fut.set_exception(e)

    def submit(self, fn) -> Future:
        fut: Future = Future()
        self._q.put((fn, fut))
        return fut

    def stop(self):
        self._q.put((None, None))


def find_free_ports(n: int) -> list[int]:
    socks, ports = [], []
    for _ in range(n):
        s = socket.socket()
        s.bind(("", 0))
        socks.append(s)
        ports.append(s.getsockname()[1])
    for s in socks:
        s.close()
    return ports


def create_app() -> FastAPI:
    app = FastAPI()
    engines: dict[str, Any] = {}
    thread = EngineThread()
    forked: dict[str, subprocess.Popen] = {}
    state = {"configured": False}

    @app.get("/health")
    def health():
        return {"status": "ok", "engines": sorted(engines), "pid": os.getpid()}

    @app.post("/alloc_ports")
    async def alloc_ports(req: Request):
        body = await req.json()
        return {"ports": find_free_ports(int(body.get("count", 1)))}

    @app.post("/set_env")
    async def set_env(req: Request):
        body = await req.json()
        for k, v in body.get("env", {}).items():
            os.environ[str(k)] = str(v)
        return {"status": "ok"}

    @app.post("/configure")
    async def configure(req: Request):
        body = await req.json()
        cfg = deserialize_value(body.get("config"))
        rank = int(body.get("rank", 0))
        role = body.get("role", "worker")
        from ...utils import name_resolve, seeding

        if cfg is not None and hasattr(cfg, "cluster"):
            name_resolve.reconfigure(cfg.cluster.name_resolve)
        if cfg is not None and hasattr(cfg, "seed"):
            seeding.set_random_seed(cfg.seed, f"{role}{rank}")
        if cfg is not None and getattr(cfg, "perf_tracer", None) is not None:
            perf_tracer.configure(cfg.perf_tracer, rank, role)
        state["configured"] = True
        return {"status": "ok"}

    @app.post("/create_engine")
    async def create_engine(req: Request):
        body = await req.json()
        name = body.get("engine_name") or "default"
        path = body["engine"]
        args = deserialize_value(body.get("args", []))
        kwargs = deserialize_value(body.get("kwargs", {}))

        def make():
            mod, _, cls = path.rpartition(".")
            engines[name] = getattr(importlib.import_module(mod), cls)(*args, **kwargs)
            return True

        try:
            thread.submit(make).result()
        except Exception as e:
            raise HTTPException(status_code=500, detail=f"{type(e).__name__}: {e}\n{traceback.format_exc()}")
        return {"status": "ok", "engine_name": name}

    @app.post("/call")
    async def call(req: Request):
        body = await req.json()
        name = body.get("engine_name") or "default"
        method = body["method"]
        if name not in engines:
            raise HTTPException(status_code=404, detail=f"engine {name!r} does not exist")
        args = rtensor.localize(deserialize_value(body.get("args", [])))
        kwargs = rtensor.localize(deserialize_value(body.get("kwargs", {})))
        as_rtensor = bool(body.get("return_rtensor", False))

        def run():
            with perf_tracer.trace_scope(f"rpc.{method}", perf_tracer.Category.SCHEDULER):
                out = getattr(engines[name], method)(*args, **kwargs)
            if hasattr(out, "result") and callable(out.result):  # concurrent Future
                out = out.result()
            if out is engines[name] or out is getattr(engines[name], "engine", None):
                out = None  # fluent methods (`initialize`, `train`) return the engine: it stays in this process
            return rtensor.remotize(out) if as_rtensor else out

        try:
            out = thread.submit(run).result()
        except Exception as e:
            raise HTTPException(status_code=500, detail=f"{type(e).__name__}: {e}\n{traceback.format_exc()}")
        return {"result": serialize_value(out)}

    @app.put("/data/{shard_id}")
    async def put_data(shard_id: str, req: Request):
        rtensor.LOCAL_STORE.put(shard_id, deserialize_value(await req.json()))
        return {"status": "ok"}

    @app.get("/data/{shard_id}")
    def get_data(shard_id: str):
        try:
            return serialize_value(rtensor.LOCAL_STORE.get(shard_id))
        except KeyError:
            raise HTTPException(status_code=404, detail=f"shard {shard_id} not found")

    @app.post("/data/batch")
    async def get_batch(req: Request):
        ids = (await req.json()).get("shard_ids", [])
        try:
            return {"tensors": [serialize_value(rtensor.LOCAL_STORE.get(i)) for i in ids]}
        except KeyError as e:
            raise HTTPException(status_code=404, detail=f"shard {e} not found")

    @app.post("/data/clear")
    async def clear_data(req: Request):
        body = await req.json() if await req.body() else {}
        ids = body.get("shard_ids")
        if ids is None:
            return {"cleared": rtensor.LOCAL_STORE.clear()}
        rtensor.LOCAL_STORE.delete(ids)
        return {"cleared": len(ids)}

    @app.post("/fork")
    async def fork(req: Request):
        body = await req.json()
        port = find_free_ports(1)[0]
        cmd = body.get("command") or f"{sys.executable} -m areal_b200.infra.rpc.rpc_server"
        env = dict(os.environ, **{str(k): str(v) for k, v in body.get("env", {}).items()})
        p = subprocess.Popen(cmd.split() + ["--port", str(port), "--host", body.get("host", "127.0.0.1")], env=env)
        wid = body.get("worker_id", f"fork-{p.pid}")
        forked[wid] = p
        return {"worker_id": wid, "port": port, "pid": p.pid}

    @app.post("/kill_forked_worker")
    async def kill_forked(req: Request):
        wid = (await req.json())["worker_id"]
        p = forked.pop(wid, None)
        if p is None:
            raise HTTPException(status_code=404, detail=f"no forked worker {wid}")
        p.terminate()
        try:
            p.wait(timeout=10)
        except subprocess.TimeoutExpired:
            p.kill()
        return {"status": "ok"}

    app.state.engines = engines
    app.state.engine_thread = thread
    return app


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=0)
    ap.add_argument("--name-key", default=None, help="name_resolve key under which to publish host:port")
    ap.add_argument("--nfs-record-root", default=None)
    args = ap.parse_args(argv)
    port = args.port or find_free_ports(1)[0]
    rtensor.set_local_addr(f"{args.host}:{port}")
    if args.name_key:
        from ...api.cli_args import NameResolveConfig
        from ...utils import name_resolve

        name_resolve.reconfigure(NameResolveConfig(type="nfs", nfs_record_root=args.nfs_record_root or
                                                   "/tmp/areal/name_resolve"))
        name_resolve.add(args.name_key, f"{args.host}:{port}", replace=True)
    logging.suppress_http_loggers()
    signal.signal(signal.SIGTERM, lambda *_: os._exit(0))
    uvicorn.run(create_app(), host=args.host, port=port, log_level="warning")


if __name__ == "__main__":
    main()
