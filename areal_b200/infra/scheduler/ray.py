"""Ray scheduler: workers are Ray actors (one per replica, placed through a placement group) that
run the worker RPC server in a thread and report their address; engine calls then go over the
same HTTP protocol as with the local scheduler. Ray is optional: constructing the scheduler
without it raises an ImportError that says so.

Counterpart of areal/infra/scheduler/ray.py:58-866 in the reference.
"""

from __future__ import annotations

import time

from ...api.cli_args import SchedulingSpec
from ...api.scheduler_api import Job, Worker
from ...utils import logging
from .exceptions import WorkerCreationError
from .local import LocalScheduler, _WorkerInfo

logger = logging.getLogger("RayScheduler")


def _require_ray():
    try:
        import ray  # noqa: F401

        return ray
    except ImportError as e:  # pragma: no cover - depends on the environment
        raise ImportError("RayScheduler needs the 'ray' package, which is not installed in this environment; "
                          "use LocalScheduler or SlurmScheduler, or install ray") from e


def placement_bundles(job: Job) -> list[dict[str, float]]:
    """One bundle per replica with the CPUs / GPUs / memory of its scheduling spec."""
    specs = job.tasks or [SchedulingSpec()]
    out = []
    for i in range(job.replicas):
        s = specs[i] if len(specs) == job.replicas else specs[0]
        b = {"CPU": float(s.cpu), "memory": float(s.mem) * (1 << 30)}
        if s.gpu:
            b["GPU"] = float(s.gpu)
        out.append(b)
    return out


class RayScheduler(LocalScheduler):
    def __init__(self, startup_timeout: float = 300.0, **kw):
        self.ray = _require_ray()
        super().__init__(gpu_devices=[], startup_timeout=startup_timeout, **kw)
        if not self.ray.is_initialized():
            self.ray.init(ignore_reinit_error=True)
        self._actors: dict[str, list] = {}
        self._pgs: dict[str, object] = {}

    def create_workers(self, job: Job, *args, **kwargs) -> list[str]:
        ray = self.ray
        role = job.role
        if role in self._workers:
            raise WorkerCreationError(role, "role already exists", "delete it first")
        from ray.util.placement_group import placement_group
        from ray.util.scheduling_strategies import PlacementGroupSchedulingStrategy

        bundles = placement_bundles(job)
        strategy = "PACK" if (job.tasks and job.tasks[0].ray_placement_strategy == "shared") else "SPREAD"
        pg = placement_group(bundles, strategy=strategy)
        ray.get(pg.ready(), timeout=self.startup_timeout)

        @ray.remote
        class _RpcWorker:
            def start(self, env):
                import os
                import socket
                import threading

                os.environ.update(env)
                from areal_b200.infra.rpc import rpc_server, rtensor

                port = rpc_server.find_free_ports(1)[0]
                host = socket.gethostbyname(socket.gethostname())
                rtensor.set_local_addr(f"{host}:{port}")
                import uvicorn

                t = threading.Thread(target=lambda: uvicorn.run(rpc_server.create_app(), host="0.0.0.0", port=port,
                                                                log_level="warning"), daemon=True)
                t.start()
                return host, port

        actors, infos = [], []
        for i, b in enumerate(bundles):
            a = _RpcWorker.options(num_cpus=b["CPU"], num_gpus=b.get("GPU", 0),
                                   scheduling_strategy=PlacementGroupSchedulingStrategy(pg, i)).remote()
            spec = (job.tasks[i] if len(job.tasks) == job.replicas else job.tasks[0]) if job.tasks else SchedulingSpec()
            host, port = ray.get(a.start.remote({str(k): str(v) for k, v in (spec.env_vars or {}).items()}))
            actors.append(a)
            infos.append(_WorkerInfo(Worker(id=f"{role}/{i}", ip=host, worker_ports=[str(port)]), None, role))
        self._actors[role], self._pgs[role], self._workers[role] = actors, pg, infos
        for info in infos:
            self._by_id[info.worker.id] = info
        return [i.worker.id for i in infos]

    def _check_alive(self, info: _WorkerInfo):
        pass  # a dead actor shows up as a failed health check / engine call

    def _terminate(self, info: _WorkerInfo):
        for a in self._actors.pop(info.role, []):
            try:
                self.ray.kill(a)
            except Exception:
                pass
        pg = self._pgs.pop(info.role, None)
        if pg is not None:
            from ray.util.placement_group import remove_placement_group

            remove_placement_group(pg)
