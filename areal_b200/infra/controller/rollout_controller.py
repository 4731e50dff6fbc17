"""Single-controller stand-in for the rollout side.

Rollout engines live in worker processes (one per data-parallel replica). The
controller keeps the *global* staleness accounting, spreads episodes over the
replicas round-robin, collects finished trajectories, fans out pause / resume /
weight updates / version changes and merges the workers' streaming statistics by
their counts (role of areal/infra/controller/rollout_controller.py:72-1130).
"""

from __future__ import annotations

import asyncio
import itertools
import threading
import time
from typing import Any

from ...api.alloc_mode import ModelAllocation
from ...api.cli_args import InferenceEngineConfig, SchedulingSpec
from ...api.io_struct import WeightUpdateMeta
from ...api.scheduler_api import Job, Scheduler, Worker
from ...utils import logging, stats_tracker
from ...utils.data import concat_padded_tensors, cycle_dataloader
from ..rpc.rtensor import localize
from ..staleness_manager import StalenessManager

logger = logging.getLogger("RolloutController")


class RolloutController:
    def __init__(self, engine: str | type, config: InferenceEngineConfig, scheduler: Scheduler):
        self.engine_path = engine if isinstance(engine, str) else f"{engine.__module__}.{engine.__qualname__}"
        self.config = config
        self.scheduler = scheduler
        self.workers: list[Worker] = []
        self.role = "rollout"
        self._version = 0
        self._rr = itertools.count()
        self._pending: list[tuple[int, str]] = []  # (task id, worker id)
        self._ids = itertools.count(1)
        self._data_iter = None
        self.staleness: StalenessManager | None = None
        self._lock = threading.Lock()
        self._paused = False
        self._failures_in_a_row = 0
        self._ready: list[dict[str, Any]] = []

    def get_version(self) -> int:
        return self._version

    def initialize(self, role: str = "rollout", alloc_mode: ModelAllocation | None = None, **kwargs):
        self.role = role
        alloc = alloc_mode or ModelAllocation.from_str(self.config.backend)
        replicas = alloc.parallel.dp_size
        spec = (list(self.config.scheduling_spec) or [SchedulingSpec()])[0]
        self.scheduler.create_workers(Job(replicas=replicas, tasks=[spec], role=role,
                                          scheduling_strategy=self.config.scheduling_strategy))
        self.workers = self.scheduler.get_workers(role, timeout=self.config.setup_timeout)
        bs = self.config.consumer_batch_size
        conc = self.config.max_concurrent_rollouts or bs
        self.staleness = StalenessManager(self, conc, bs, self.config.max_head_offpolicyness)

        async def setup():
            await asyncio.gather(*[self.scheduler.create_engine(w.id, self.engine_path, self.config,
                                                                engine_name=role) for w in self.workers])
            await asyncio.gather(*[self.scheduler.async_call_engine(
                w.id, "initialize", role, train_data_parallel_size=replicas, **kwargs) for w in self.workers])

        asyncio.run(setup())
        return self

    def destroy(self):
        try:
            self.scheduler.delete_workers(self.role)
        except Exception as e:
            logger.warning(f"could not delete rollout workers: {e}")

    def _fanout(self, method: str, *args, **kwargs) -> list[Any]:
        async def run():
            return await asyncio.gather(*[self.scheduler.async_call_engine(w.id, method, self.role, *args, **kwargs)
                                          for w in self.workers])

        return asyncio.run(run())

    # -------------------------------------------------------------- rollouts
    def get_capacity(self) -> int:
        return self.staleness.get_capacity()

    def submit(self, data: dict[str, Any], workflow=None, workflow_kwargs=None, should_accept_fn=None,
               group_size: int = 1, **kw) -> int:
        """Workflows cross the process boundary as import paths (+ kwargs)."""
        if not isinstance(workflow, str):
            workflow = f"{workflow.__module__}.{workflow.__qualname__}" if isinstance(workflow, type) else workflow
        w = self.workers[next(self._rr) % len(self.workers)]
        tid = next(self._ids)
        self.staleness.on_rollout_enqueued()
        self.staleness.on_rollout_submitted()
        self.scheduler.call_engine(w.id, "submit", self.role, data, workflow, workflow_kwargs, should_accept_fn,
                                   group_size, task_id=tid)
        with self._lock:
            self._pending.append((tid, w.id))
        return tid

    def wait(self, count: int, timeout: float | None = None, raise_timeout: bool = True):
        deadline = None if timeout is None else time.monotonic() + timeout
        got = self._ready  # trajectories collected by earlier calls that timed out stay here
        while len(got) < count:
            progressed = False
            with self._lock:
                pending = list(self._pending)
            for tid, wid in pending:
                if len(got) >= count:
                    break
                state, r = self.scheduler.call_engine(wid, "poll_task", self.role, tid)
                if state == "running":
                    continue
                with self._lock:
                    self._pending.remove((tid, wid))
                progressed = True
                if state == "done":
                    self._failures_in_a_row = 0
                    self.staleness.on_rollout_accepted()
                    got.append(localize(r))
                    continue
                # dropped by the workflow / acceptance filter, or the episode raised: the sample will never
                # arrive; free its slot so that prepare_batch submits a replacement
                self.staleness.on_rollout_rejected()
                if state == "failed":
                    self._failures_in_a_row += 1
                    logger.warning(f"rollout task {tid} on {wid} failed: {r}")
                    if self._failures_in_a_row >= 16:
                        raise RuntimeError(f"{self._failures_in_a_row} rollout episodes failed in a row; last: {r}")
            if len(got) >= count:
                break
            if deadline is not None and time.monotonic() > deadline:
                if raise_timeout:
                    raise TimeoutError(f"{len(got)}/{count} rollouts within {timeout}s")
                return None
            if not progressed:
                time.sleep(0.01)
        take, self._ready = got[:count], got[count:]
        return concat_padded_tensors(take)

    def rollout_batch(self, data: list[dict[str, Any]], workflow=None, workflow_kwargs=None,
                      should_accept_fn=None, group_size: int = 1):
        for d in data:
            self.submit(d, workflow, workflow_kwargs, should_accept_fn, group_size)
        return self.wait(len(data), timeout=self.config.request_timeout)

    def prepare_batch(self, dataloader, workflow=None, workflow_kwargs=None, should_accept_fn=None,
                      group_size: int = 1, dynamic_bs: bool = False):
        if self._data_iter is None:
            self._data_iter = cycle_dataloader(dataloader)
        bs = getattr(dataloader, "batch_size", None) or self.config.consumer_batch_size
        while True:
            while not self._paused and self.get_capacity() >= bs:
                items = next(self._data_iter)
                for it in (items if isinstance(items, list) else [items]):
                    self.submit(it, workflow, workflow_kwargs, should_accept_fn, group_size)
            out = self.wait(bs, timeout=0.5, raise_timeout=False)
            if out is not None:
                return out

    # ---------------------------------------------------------------- control
    def pause(self):
        self._paused = True
        self._fanout("pause")

    def resume(self):
        self._paused = False
        self._fanout("resume")

    def pause_generation(self):
        self._fanout("pause_generation")

    def continue_generation(self):
        self._fanout("continue_generation")

    def set_version(self, version: int):
        self._version = version
        self._fanout("set_version", version)

    def update_weights_from_disk(self, meta: WeightUpdateMeta):
        from concurrent.futures import Future

        self._fanout("update_weights_from_disk", meta)
        f: Future = Future()
        f.set_result(None)
        return f

    def export_stats(self) -> dict[str, float]:
        merged = stats_tracker.merge_scalar_stats(self._fanout("export_stats"))
        s = self.staleness.get_stats()
        merged.update({"rollout_controller/accepted": float(s.accepted), "rollout_controller/running": float(s.running)})
        return merged
