"""Local scheduler: workers are subprocesses on this machine.

``create_workers`` starts ``python -m areal_b200.infra.rpc.rpc_server`` per
replica with GPUs assigned round-robin (``CUDA_VISIBLE_DEVICES``) or shared with
the worker they are colocated with; ``get_workers`` waits for ``/health``;
``create_engine`` / ``call_engine`` / ``async_call_engine`` talk to the workers'
RPC endpoints with exponential-backoff retries and watch for dead processes
(role of areal/infra/scheduler/local.py:203-1540 in the reference).
"""

from __future__ import annotations

import asyncio
import os
import subprocess
import sys
import time
from dataclasses import dataclass, field
from typing import Any

import aiohttp
import requests

from ...api.cli_args import SchedulingStrategy
from ...api.scheduler_api import Job, Scheduler, Worker
from ...utils import logging
from ..rpc.rpc_server import find_free_ports
from ..rpc.serialization import deserialize_value, serialize_value
from .exceptions import (EngineCallError, EngineCreationError, GPUAllocationError, RPCConnectionError,
                         WorkerCreationError, WorkerFailedError, WorkerNotFoundError, WorkerTimeoutError)

logger = logging.getLogger("LocalScheduler")


@dataclass
class _WorkerInfo:
    worker: Worker
    process: subprocess.Popen | None
    role: str
    gpus: list[int] = field(default_factory=list)
    log_path: str | None = None
    env: dict[str, str] = field(default_factory=dict)


class LocalScheduler(Scheduler):
    def __init__(self, gpu_devices: list[int] | None = None, log_dir: str | None = None,
                 startup_timeout: float = 60.0, health_interval: float = 0.2, n_gpus_per_node: int | None = None,
                 max_retries: int = 3, retry_backoff: float = 0.2, worker_command: str | None = None):
        if gpu_devices is None:
            env = os.environ.get("CUDA_VISIBLE_DEVICES")
            if env:
                gpu_devices = [int(x) for x in env.split(",") if x.strip() != ""]
            else:
                n = n_gpus_per_node
                if n is None:
                    try:
                        import torch

                        n = torch.cuda.device_count()
                    except Exception:
                        n = 0
                gpu_devices = list(range(n))
        self.gpu_devices = gpu_devices
        self._gpu_cursor = 0
        self.log_dir = log_dir or "/tmp/areal_b200/scheduler_logs"
        os.makedirs(self.log_dir, exist_ok=True)
        self.startup_timeout, self.health_interval = startup_timeout, health_interval
        self.max_retries, self.retry_backoff = max_retries, retry_backoff
        self.worker_command = worker_command or f"{sys.executable} -m areal_b200.infra.rpc.rpc_server"
        self._workers: dict[str, list[_WorkerInfo]] = {}
        self._by_id: dict[str, _WorkerInfo] = {}

    # ---------------------------------------------------------------- GPUs
    def _allocate_gpus(self, n: int) -> list[int]:
        if n == 0:
            return []
        if not self.gpu_devices:
            raise GPUAllocationError("no GPU available on this machine")
        if n > len(self.gpu_devices):
            raise GPUAllocationError(f"requested {n} GPUs, only {len(self.gpu_devices)} exist")
        out = []
        for _ in range(n):
            out.append(self.gpu_devices[self._gpu_cursor % len(self.gpu_devices)])
            self._gpu_cursor += 1
        return out

    # -------------------------------------------------------------- workers
    def create_workers(self, job: Job, *args, **kwargs) -> list[str]:
        role = job.role
        if role in self._workers:
            raise WorkerCreationError(role, "role already exists", "delete it first")
        if job.replicas <= 0:
            raise WorkerCreationError(role, "invalid configuration", "replicas must be positive")
        specs = job.tasks or []
        if len(specs) not in (0, 1, job.replicas):
            raise WorkerCreationError(role, "invalid configuration",
                                      f"got {len(specs)} scheduling specs for {job.replicas} replicas")
        strat = job.scheduling_strategy or SchedulingStrategy()
        target_infos = None
        if strat.type == "colocation":
            if not strat.target or strat.target not in self._workers:
                raise WorkerCreationError(role, "colocation target missing", f"target={strat.target!r}")
            target_infos = self._workers[strat.target]
            if len(target_infos) != job.replicas:
                raise WorkerCreationError(role, "replica mismatch",
                                          f"target has {len(target_infos)} workers, requested {job.replicas}")
        infos = []
        try:
            for i in range(job.replicas):
                spec = specs[i] if len(specs) == job.replicas else (specs[0] if specs else None)
                gpus = target_infos[i].gpus if target_infos is not None else \
                    self._allocate_gpus(spec.gpu if spec is not None else 0)
                port = find_free_ports(1)[0]
                wid = f"{role}/{i}"
                env = dict(os.environ)
                env["CUDA_VISIBLE_DEVICES"] = ",".join(map(str, gpus))
                env["AREAL_WORKER_ID"] = wid
                if spec is not None:
                    env.update({str(k): str(v) for k, v in (spec.env_vars or {}).items()})
                cmd = (spec.cmd if (spec is not None and spec.cmd) else self.worker_command).split()
                cmd += ["--host", "127.0.0.1", "--port", str(port)]
                log_path = os.path.join(self.log_dir, f"{role.replace('/', '_')}_{i}.log")
                logf = open(log_path, "w")
                proc = subprocess.Popen(cmd, env=env, stdout=logf, stderr=subprocess.STDOUT)
                info = _WorkerInfo(Worker(id=wid, ip="127.0.0.1", worker_ports=[str(port)]), proc, role, gpus,
                                   log_path)
                infos.append(info)
        except Exception as e:
            for info in infos:
                self._terminate(info)
            if isinstance(e, (WorkerCreationError, GPUAllocationError)):
                raise
            raise WorkerCreationError(role, "spawn failed", str(e)) from e
        self._workers[role] = infos
        for info in infos:
            self._by_id[info.worker.id] = info
        return [i.worker.id for i in infos]

    def _addr(self, info: _WorkerInfo) -> str:
        return f"{info.worker.ip}:{info.worker.worker_ports[0]}"

    def _check_alive(self, info: _WorkerInfo):
        if info.process is not None and info.process.poll() is not None:
            tail = ""
            if info.log_path and os.path.exists(info.log_path):
                with open(info.log_path) as f:
                    tail = f.read()[-2000:]
            raise WorkerFailedError(info.worker.id, info.process.returncode, tail)

    def get_workers(self, role: str, timeout: float | None = None) -> list[Worker]:
        if role not in self._workers:
            raise WorkerNotFoundError(role)
        deadline = time.monotonic() + (timeout if timeout is not None else self.startup_timeout)
        pending = list(self._workers[role])
        while pending:
            for info in list(pending):
                self._check_alive(info)
                try:
                    r = requests.get(f"http://{self._addr(info)}/health", timeout=2)
                    if r.status_code == 200:
                        pending.remove(info)
                except requests.RequestException:
                    pass
            if pending:
                if time.monotonic() > deadline:
                    raise WorkerTimeoutError(role, timeout if timeout is not None else self.startup_timeout)
                time.sleep(self.health_interval)
        return [i.worker for i in self._workers[role]]

    def _terminate(self, info: _WorkerInfo):
        p = info.process
        if p is None or p.poll() is not None:
            return
        p.terminate()
        try:
            p.wait(timeout=5)
        except subprocess.TimeoutExpired:
            p.kill()
            p.wait(timeout=5)

    def delete_workers(self, role: str | None = None):
        roles = [role] if role is not None else list(self._workers)
        for r in roles:
            if r not in self._workers:
                raise WorkerNotFoundError(r)
            for info in self._workers.pop(r):
                self._terminate(info)
                self._by_id.pop(info.worker.id, None)

    def fork_workers(self, role: str, target_role: str, command: str | None = None) -> list[str]:
        """Asks every worker of ``target_role`` to fork a sibling process (same GPUs) for ``role``."""
        if target_role not in self._workers:
            raise WorkerNotFoundError(target_role)
        infos = []
        for i, t in enumerate(self._workers[target_role]):
            r = requests.post(f"http://{self._addr(t)}/fork",
                              json={"worker_id": f"{role}/{i}", "command": command}, timeout=30)
            if r.status_code != 200:
                raise WorkerCreationError(role, "fork failed", r.text)
            d = r.json()
            infos.append(_WorkerInfo(Worker(id=d["worker_id"], ip="127.0.0.1", worker_ports=[str(d["port"])]),
                                     None, role, t.gpus))
        self._workers[role] = infos
        for info in infos:
            self._by_id[info.worker.id] = info
        return [i.worker.id for i in infos]

    # -------------------------------------------------------------- engines
    def _info(self, worker_id: str) -> _WorkerInfo:
        if worker_id not in self._by_id:
            raise WorkerNotFoundError(worker_id)
        return self._by_id[worker_id]

    async def set_worker_env(self, worker_id: str, env: dict[str, str]) -> None:
        info = self._info(worker_id)
        async with aiohttp.ClientSession() as s:
            async with s.post(f"http://{self._addr(info)}/set_env", json={"env": env}) as r:
                if r.status != 200:
                    raise EngineCallError(worker_id, "set_env", await r.text())

    async def create_engine(self, worker_id: str, engine: str, *args, engine_name: str | None = None, **kwargs):
        info = self._info(worker_id)
        self._check_alive(info)
        payload = {"engine": engine, "engine_name": engine_name, "args": serialize_value(list(args)),
                   "kwargs": serialize_value(kwargs)}
        try:
            async with aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=3600)) as s:
                async with s.post(f"http://{self._addr(info)}/create_engine", json=payload) as r:
                    if r.status != 200:
                        raise EngineCreationError(worker_id, await r.text(), r.status)
                    return await r.json()
        except aiohttp.ClientError as e:
            self._check_alive(info)
            raise RPCConnectionError(worker_id, self._addr(info), str(e)) from e

    def _payload(self, method, engine_name, args, kwargs, return_rtensor=False):
        return {"method": method, "engine_name": engine_name, "args": serialize_value(list(args)),
                "kwargs": serialize_value(kwargs), "return_rtensor": return_rtensor}

    def call_engine(self, worker_id: str, method: str, engine_name: str | None = None, *args,
                    max_retries: int | None = None, return_rtensor: bool = False, http_timeout: float = 7200.0,
                    **kwargs) -> Any:
        info = self._info(worker_id)
        payload = self._payload(method, engine_name, args, kwargs, return_rtensor)
        retries = self.max_retries if max_retries is None else max_retries
        last = ""
        for attempt in range(1, retries + 1):
            self._check_alive(info)
            try:
                r = requests.post(f"http://{self._addr(info)}/call", json=payload, timeout=http_timeout)
                if r.status_code == 200:
                    return deserialize_value(r.json()["result"])
                last = r.text
                if 400 <= r.status_code < 500 or r.status_code == 500:
                    # the engine itself raised: retrying cannot help
                    raise EngineCallError(worker_id, method, last, attempt)
            except requests.RequestException as e:
                last = str(e)
            if attempt < retries:
                time.sleep(self.retry_backoff * 2 ** (attempt - 1))
        self._check_alive(info)
        raise EngineCallError(worker_id, method, last, retries)

    async def async_call_engine(self, worker_id: str, method: str, engine_name: str | None = None, *args,
                                max_retries: int | None = None, return_rtensor: bool = False,
                                http_timeout: float = 7200.0, **kwargs) -> Any:
        info = self._info(worker_id)
        payload = self._payload(method, engine_name, args, kwargs, return_rtensor)
        retries = self.max_retries if max_retries is None else max_retries
        last = ""
        for attempt in range(1, retries + 1):
            self._check_alive(info)
            try:
                async with aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=http_timeout)) as s:
                    async with s.post(f"http://{self._addr(info)}/call", json=payload) as r:
                        if r.status == 200:
                            return deserialize_value((await r.json())["result"])
                        last = await r.text()
                        raise EngineCallError(worker_id, method, last, attempt)
            except aiohttp.ClientError as e:
                last = str(e)
            if attempt < retries:
                await asyncio.sleep(self.retry_backoff * 2 ** (attempt - 1))
        self._check_alive(info)
        raise EngineCallError(worker_id, method, last, retries)

    def __del__(self):
        try:
            for infos in self._workers.values():
                for info in infos:
                    self._terminate(info)
        except Exception:
            pass
