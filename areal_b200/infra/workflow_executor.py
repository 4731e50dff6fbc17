"""Runs rollout workflows asynchronously under a staleness bound and hands
finished trajectories to the trainer.

``submit`` enqueues one episode; a background asyncio runner starts it as soon as
the :class:`StalenessManager` grants capacity; finished episodes are accepted or
rejected (``None`` result or ``should_accept_fn``) and collected by ``wait``.
``prepare_batch`` keeps the pipeline filled from a dataloader and returns one
training batch; ``rollout_batch`` is the synchronous variant.

Workflows may be given as an instance, a class (+kwargs), an import path, or any
object with ``async run(data, **extra)`` (agent workflow, run through the
OpenAI-compatible proxy). ``group_size > 1`` runs the episode that many times
concurrently and concatenates the results (GRPO groups stay together).

Reference: areal/infra/workflow_executor.py:47-1372,
areal/infra/remote_inf_engine.py:70,541-655.
"""

from __future__ import annotations

import asyncio
import importlib
import itertools
import random
import threading
import time
from typing import Any, Callable

from ..utils.dynamic_import import import_from_string

import torch

from ..api.cli_args import InferenceEngineConfig
from ..api.workflow_api import RolloutWorkflow
from ..utils import logging
from ..utils.data import concat_padded_tensors, cycle_dataloader
from .async_task_runner import AsyncTaskRunner, TaskQueueFullError, TimedResult
from .staleness_manager import StalenessManager

logger = logging.getLogger("WorkflowExecutor")

REQUIRED_KEYS = ("input_ids", "attention_mask")


def check_trajectory_format(traj: Any, batch_size: int | None = None) -> bool:
    """Validates a trajectory: ``None`` (rejected) or a dict of tensors whose leading
    dimension agrees, containing ``input_ids`` and ``attention_mask`` of equal shape."""
    if traj is None:
        return True
    if not isinstance(traj, dict):
        raise ValueError(f"trajectory must be a dict or None, got {type(traj).__name__}")
    if not traj:
        raise ValueError("trajectory dict is empty")
    first = next(iter(traj.values()))
    if not torch.is_tensor(first):
        # dict of interactions: each must expose to_tensor_dict()
        for k, v in traj.items():
            if not hasattr(v, "to_tensor_dict"):
                raise ValueError(f"interaction {k!r} has no to_tensor_dict()")
        return True
    for k in REQUIRED_KEYS:
        if k not in traj:
            raise ValueError(f"trajectory lacks required key {k!r}")
    ids, mask = traj["input_ids"], traj["attention_mask"]
    if ids.dim() != 2 or ids.shape != mask.shape:
        raise ValueError(f"input_ids {tuple(ids.shape)} and attention_mask {tuple(mask.shape)} must be equal 2-D shapes")
    B, L = ids.shape
    if batch_size is not None and B != batch_size:
        raise ValueError(f"expected batch size {batch_size}, got {B}")
    for k, v in traj.items():
        if torch.is_tensor(v) and v.dim() >= 1 and v.shape[0] != B:
            raise ValueError(f"{k}: leading dimension {v.shape[0]} != batch size {B}")
        if torch.is_tensor(v) and v.dim() >= 2 and k in ("loss_mask", "logprobs", "versions") and v.shape[1] != L:
            raise ValueError(f"{k}: sequence dimension {v.shape[1]} != {L}")
    return True


def _to_tensor_dict(traj: Any) -> dict[str, Any] | None:
    if traj is None:
        return None
    first = next(iter(traj.values()), None)
    if torch.is_tensor(first) or not hasattr(first, "to_tensor_dict"):
        return traj
    return concat_padded_tensors([v.to_tensor_dict() for v in traj.values()])


class GroupedRolloutWorkflow(RolloutWorkflow):
    """Runs the wrapped workflow ``group_size`` times concurrently on the same item."""

    def __init__(self, workflow: RolloutWorkflow, group_size: int):
        self.workflow, self.group_size = workflow, group_size

    async def arun_episode(self, engine, data):
        results = await asyncio.gather(*[self.workflow.arun_episode(engine, data) for _ in range(self.group_size)])
        results = [_to_tensor_dict(r) for r in results if r is not None]
        if not results:
            return None
        return concat_padded_tensors(results)


def resolve_workflow(workflow: Any, workflow_kwargs: dict | None, group_size: int = 1,
                     proxy_factory: Callable | None = None) -> RolloutWorkflow:
    """Accepts an instance, a class, an import path, or an agent with ``async run``."""
    kwargs = workflow_kwargs or {}
    if isinstance(workflow, str):
        workflow = import_from_string(workflow)
    if isinstance(workflow, type):
        workflow = workflow(**kwargs)
    if not isinstance(workflow, RolloutWorkflow):
        if hasattr(workflow, "run") and asyncio.iscoroutinefunction(workflow.run):
            if proxy_factory is None:
                from ..openai.proxy.workflow import OpenAIProxyWorkflow

                workflow = OpenAIProxyWorkflow(agent=workflow)
            else:
                workflow = proxy_factory(workflow)
        else:
            raise TypeError(f"cannot interpret {workflow!r} as a rollout workflow")
    if group_size > 1:
        workflow = GroupedRolloutWorkflow(workflow, group_size)
    return workflow


class WorkflowExecutor:
    MAX_CONSECUTIVE_FAILURES = 64

    def __init__(self, config: InferenceEngineConfig, engine):
        self.config = config
        self.engine = engine
        self.runner: AsyncTaskRunner | None = None
        self.staleness: StalenessManager | None = None
        self._results: list[TimedResult] = []
        self._by_task: dict[int, TimedResult] = {}
        self._ids = itertools.count(1)
        self._lock = threading.Lock()
        self._data_iter = None
        self._rng = random.Random(0)
        self._n_failed = 0
        self._consecutive_failures = 0  # episodes that raised since the last one that did not
        self._last_error = None
        self._eval_runner: AsyncTaskRunner | None = None  # evaluation episodes: no staleness gate, own queue
        self._eval_tasks: set[int] = set()

    def initialize(self, train_data_parallel_size: int | None = None):
        cfg = self.config
        dp = max(train_data_parallel_size or 1, 1)
        bs = max(cfg.consumer_batch_size // dp, 1)
        max_conc = cfg.max_concurrent_rollouts or cfg.consumer_batch_size
        max_conc = max(max_conc // dp, 1)
        self.staleness = StalenessManager(self.engine, max_conc, bs, cfg.max_head_offpolicyness)
        qsize = cfg.queue_size or max(max_conc * 16, 1024)
        self.runner = AsyncTaskRunner(max_queue_size=qsize)
        self.runner.initialize(admit_fn=self._admit)
        return self

    def destroy(self):
        if self.runner is not None:
            self.runner.destroy()
            self.runner = None
        if self._eval_runner is not None:
            self._eval_runner.destroy()
            self._eval_runner = None

    # staleness gate: consulted by the runner thread before each task start
    def _admit(self) -> bool:
        if self.staleness.get_capacity() <= 0:
            return False
        self.staleness.on_rollout_submitted()
        return True

    def on_version_changed(self, version: int):
        pass  # capacity is recomputed from the engine's version on every admit

    def get_capacity(self) -> int:
        return self.staleness.get_capacity()

    def pause(self):
        self.runner.pause()

    def resume(self):
        self.runner.resume()

    # ------------------------------------------------------------------ submit
    def submit(self, data: dict[str, Any], workflow=None, workflow_kwargs=None, should_accept_fn=None,
               group_size: int = 1, task_id: int | None = None, is_eval: bool = False) -> int:
        wf = resolve_workflow(workflow, workflow_kwargs, group_size)
        if isinstance(should_accept_fn, str):
            should_accept_fn = import_from_string(should_accept_fn)
        tid = task_id if task_id is not None else next(self._ids)
        if is_eval:
            # evaluation samples are not training data: they do not count against the staleness budget and must
            # not queue behind training episodes that wait for capacity, so they run on a runner of their own
            if self._eval_runner is None:
                self._eval_runner = AsyncTaskRunner(max_queue_size=self.runner.max_queue_size)
                self._eval_runner.initialize()
            with self._lock:
                self._eval_tasks.add(tid)
            self._eval_runner.submit(self._episode, wf, data, should_accept_fn, True, task_id=tid)
            return tid
        self.staleness.on_rollout_enqueued()
        try:
            self.runner.submit(self._episode, wf, data, should_accept_fn, task_id=tid)
        except TaskQueueFullError:
            with self.staleness.lock:
                self.staleness.rollout_stat.enqueued -= 1
            raise
        return tid

    async def _episode(self, wf: RolloutWorkflow, data, should_accept_fn, is_eval: bool = False):
        from ..utils import perf_tracer

        accepted = False
        st = perf_tracer.get_session_tracer() if self.config.enable_rollout_tracing else None
        sid = st.start_session() if st is not None else None
        try:
            if st is not None:
                with st.phase(sid, "episode"):
                    traj = await wf.arun_episode(self.engine, data)
            else:
                traj = await wf.arun_episode(self.engine, data)
            if self.config.check_trajectory_format:
                check_trajectory_format(traj)
            traj = _to_tensor_dict(traj)
            accepted = traj is not None and (should_accept_fn is None or bool(should_accept_fn(traj)))
            return traj if accepted else None
        finally:
            if st is not None:
                st.end_session(sid, status="accepted" if accepted else "rejected")
            if is_eval:
                pass
            elif accepted:
                self.staleness.on_rollout_accepted()
            else:
                self.staleness.on_rollout_rejected()

    # -------------------------------------------------------------------- wait
    def _drain(self):
        for runner in (self.runner, self._eval_runner):
            while runner is not None:
                r = runner.poll()
                if r is None:
                    break
                if r.error is not None:
                    self._n_failed += 1
                    self._consecutive_failures += 1
                    self._last_error = r.error
                    with self._lock:
                        self._by_task[r.task_id] = r  # so that a caller polling this task learns that it failed
                    continue
                self._consecutive_failures = 0
                with self._lock:
                    self._by_task[r.task_id] = r
                    if r.task_id in self._eval_tasks:
                        self._eval_tasks.discard(r.task_id)  # fetched by task id only, never part of a batch
                    elif r.data is not None:
                        self._results.append(r)

    def wait(self, count: int, timeout: float | None = None, raise_timeout: bool = True):
        """Returns ``count`` accepted trajectories concatenated into one padded batch, oldest
        first then shuffled inside the batch."""
        deadline = None if timeout is None else time.monotonic() + timeout
        while True:
            self.runner.health_check()
            self._drain()
            if self._consecutive_failures >= self.MAX_CONSECUTIVE_FAILURES:
                # a workflow that raises on every episode would otherwise keep this loop waiting forever
                raise RuntimeError(f"{self._consecutive_failures} rollout episodes failed in a row; "
                                   f"last error: {self._last_error}")
            with self._lock:
                if len(self._results) >= count:
                    self._results.sort(key=lambda r: r.create_time)
                    take, self._results = self._results[:count], self._results[count:]
                    break
            if deadline is not None and time.monotonic() > deadline:
                if raise_timeout:
                    raise TimeoutError(f"timed out waiting for {count} rollouts "
                                       f"({len(self._results)} ready, {self._n_failed} failed)")
                return None
            time.sleep(0.002)
        self._rng.shuffle(take)
        for r in take:
            self._by_task.pop(r.task_id, None)
        return concat_padded_tensors([r.data for r in take])

    def wait_for_task(self, task_id: int, timeout: float | None = None, raise_timeout: bool = True):
        deadline = None if timeout is None else time.monotonic() + timeout
        while True:
            self.runner.health_check()
            self._drain()
            with self._lock:
                r = self._by_task.pop(task_id, None)
                if r is not None:
                    self._results = [x for x in self._results if x.task_id != task_id]
                    return r.data
            if deadline is not None and time.monotonic() > deadline:
                if raise_timeout:
                    raise TimeoutError(f"task {task_id} did not finish within {timeout}s")
                return None
            time.sleep(0.002)

    def poll_task(self, task_id: int) -> tuple[str, Any]:
        """Non-blocking state of one task: ``("running", None)``, ``("done", trajectory)``, ``("rejected", None)``
        (the workflow or the acceptance filter dropped the sample) or ``("failed", message)``. A finished task is
        forgotten once reported. Used by a rollout controller in another process, which must tell a sample that
        will never arrive from one that is still being generated."""
        self.runner.health_check()
        self._drain()
        with self._lock:
            r = self._by_task.pop(task_id, None)
            if r is None:
                return "running", None
            if r.error is not None:
                return "failed", f"{type(r.error).__name__}: {r.error}"
            if r.data is None:
                return "rejected", None
            self._results = [x for x in self._results if x.task_id != task_id]
            return "done", r.data

    def rollout_batch(self, data: list[dict[str, Any]], workflow=None, workflow_kwargs=None,
                      should_accept_fn=None, group_size: int = 1, is_eval: bool = False):
        """Synchronous: submits every item and waits for all accepted results. ``is_eval`` keeps the samples
        out of the staleness accounting and off the training queue."""
        tids = [self.submit(d, workflow, workflow_kwargs, should_accept_fn, group_size, is_eval=is_eval)
                for d in data]
        outs = []
        for t in tids:
            r = self.wait_for_task(t, timeout=self.config.request_timeout)
            if r is not None:
                outs.append(r)
        return concat_padded_tensors(outs) if outs else {}

    def prepare_batch(self, dataloader, workflow=None, workflow_kwargs=None, should_accept_fn=None,
                      group_size: int = 1, dynamic_bs: bool = False):
        """Asynchronous: keeps up to ``(η+1)·batch`` episodes in flight from ``dataloader`` and
        returns as soon as one batch of accepted trajectories is available."""
        if self._data_iter is None:
            self._data_iter = cycle_dataloader(dataloader)
        bs = getattr(dataloader, "batch_size", None) or self.staleness.consumer_batch_size
        while True:
            # top up the queue: capacity says how many may *run*; also keep one batch queued
            st = self.staleness.get_stats()
            if (self.staleness.get_capacity() + bs > st.enqueued
                    and self.runner.get_input_queue_size() + bs <= self.runner.max_queue_size):
                items = next(self._data_iter)
                items = items if isinstance(items, list) else [items]
                for item in items:
                    self.submit(item, workflow, workflow_kwargs, should_accept_fn, group_size)
            out = self.wait(bs, timeout=0.05, raise_timeout=False)
            if out is not None:
                return out

    def export_stats(self) -> dict[str, float]:
        s = self.staleness.get_stats()
        return {"rollout/accepted": float(s.accepted), "rollout/running": float(s.running),
                "rollout/enqueued": float(s.enqueued), "rollout/rejected": float(s.rejected),
                "rollout/failed": float(self._n_failed)}
