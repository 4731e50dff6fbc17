"""Async task runner and workflow executor (staleness gate, accept/reject, ordering)."""
import asyncio
import threading
import time

import pytest
import torch

from areal_b200.api.cli_args import InferenceEngineConfig
from areal_b200.api.workflow_api import RolloutWorkflow
from areal_b200.infra.async_task_runner import AsyncTaskRunner, TaskQueueFullError
from areal_b200.infra.workflow_executor import (GroupedRolloutWorkflow, WorkflowExecutor, check_trajectory_format,
                                                resolve_workflow)


def test_runner_submit_wait_pause_and_failures():
    r = AsyncTaskRunner(max_queue_size=4)
    r.initialize()

    async def work(x, delay=0.0):
        await asyncio.sleep(delay)
        if x < 0:
            raise ValueError("boom")
        return x * 2

    ids = [r.submit(work, i) for i in range(3)]
    got = sorted(x.data for x in r.wait(3, timeout=5))
    assert got == [0, 2, 4] and len(set(ids)) == 3
    r.pause()
    r.submit(work, 5)
    time.sleep(0.1)
    assert r.get_output_queue_size() == 0 and r.get_input_queue_size() == 1
    with pytest.raises(TimeoutError):
        r.wait(1, timeout=0.1)
    r.resume()
    assert r.wait(1, timeout=5)[0].data == 10
    r.submit(work, -1)
    res = r.wait(1, timeout=5)[0]
    assert res.data is None and isinstance(res.error, ValueError)
    r.pause()
    for i in range(4):
        r.submit(work, i)
    with pytest.raises(TaskQueueFullError):
        r.submit(work, 9)
    r.destroy()
    with pytest.raises(RuntimeError):
        r.submit(work, 1)


class FakeEngine:
    def __init__(self):
        self.version = 0

    def get_version(self):
        return self.version


class CountingWorkflow(RolloutWorkflow):
    started = 0
    lock = threading.Lock()

    def __init__(self, reject_odd=False, delay=0.01):
        self.reject_odd, self.delay = reject_odd, delay

    async def arun_episode(self, engine, data):
        with CountingWorkflow.lock:
            CountingWorkflow.started += 1
        await asyncio.sleep(self.delay)
        if self.reject_odd and data["i"] % 2:
            return None
        n = 3 + data["i"] % 3
        return dict(input_ids=torch.full((1, n), data["i"]), attention_mask=torch.ones(1, n, dtype=torch.bool),
                    rewards=torch.tensor([float(data["i"])]), versions=torch.full((1, n), engine.get_version()))


def _executor(bs=4, eta=0, conc=64):
    eng = FakeEngine()
    cfg = InferenceEngineConfig(backend="native:d1", consumer_batch_size=bs, max_head_offpolicyness=eta,
                                max_concurrent_rollouts=conc)
    ex = WorkflowExecutor(cfg, eng).initialize()
    return eng, ex


def test_executor_staleness_gate_blocks_until_version_advances():
    CountingWorkflow.started = 0
    eng, ex = _executor(bs=4, eta=1)
    for i in range(20):
        ex.submit({"i": i}, CountingWorkflow)
    b1 = ex.wait(4, timeout=10)
    b2 = ex.wait(4, timeout=10)
    assert b1["input_ids"].shape[0] == 4 and b2["rewards"].shape == (4,)
    time.sleep(0.2)
    # (eta + version + 1) * bs = 8 episodes may start at version 0
    assert CountingWorkflow.started == 8
    assert ex.wait(1, timeout=0.2, raise_timeout=False) is None
    eng.version = 1
    b3 = ex.wait(4, timeout=10)
    assert (b3["versions"].max() == 1) and CountingWorkflow.started == 12
    st = ex.export_stats()
    assert st["rollout/accepted"] == 12 and st["rollout/enqueued"] == 8
    ex.destroy()


def test_executor_rejection_and_should_accept():
    eng, ex = _executor(bs=2, eta=100)
    for i in range(8):
        ex.submit({"i": i}, CountingWorkflow, workflow_kwargs=dict(reject_odd=True),
                  should_accept_fn=lambda t: float(t["rewards"][0]) != 4.0)
    out = ex.wait(3, timeout=10)
    assert sorted(out["rewards"].tolist()) == [0.0, 2.0, 6.0]
    time.sleep(0.1)
    st = ex.export_stats()
    assert st["rollout/accepted"] == 3 and st["rollout/rejected"] == 5 and st["rollout/running"] == 0
    ex.destroy()


def test_rollout_batch_group_and_wait_for_task():
    eng, ex = _executor(bs=2, eta=100)
    out = ex.rollout_batch([{"i": 1}, {"i": 2}], CountingWorkflow, group_size=3)
    assert out["input_ids"].shape[0] == 6 and out["attention_mask"].shape == out["input_ids"].shape
    tid = ex.submit({"i": 5}, CountingWorkflow())
    assert ex.wait_for_task(tid, timeout=5)["rewards"].tolist() == [5.0]
    ex.destroy()


def test_workflow_resolution_forms():
    wf = resolve_workflow("tests.test_async_runtime.CountingWorkflow", dict(delay=0.0))
    assert isinstance(wf, CountingWorkflow)
    assert isinstance(resolve_workflow(CountingWorkflow, None, group_size=2), GroupedRolloutWorkflow)
    inst = CountingWorkflow()
    assert resolve_workflow(inst, None) is inst
    with pytest.raises(TypeError):
        resolve_workflow(object(), None)


def test_trajectory_format_checks():
    ok = dict(input_ids=torch.zeros(2, 5, dtype=torch.long), attention_mask=torch.ones(2, 5, dtype=torch.bool),
              rewards=torch.zeros(2))
    assert check_trajectory_format(ok) and check_trajectory_format(None)
    with pytest.raises(ValueError):
        check_trajectory_format({"input_ids": torch.zeros(2, 5)})
    with pytest.raises(ValueError):
        check_trajectory_format(dict(ok, rewards=torch.zeros(3)))
    with pytest.raises(ValueError):
        check_trajectory_format(dict(ok, logprobs=torch.zeros(2, 4)))
    with pytest.raises(ValueError):
        check_trajectory_format([1, 2])
