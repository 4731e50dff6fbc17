"""Train controller over real subprocess workers with a fake CPU engine: dispatch, merge, fan-out."""
import pytest
import torch

from areal_b200.api.alloc_mode import ModelAllocation, ParallelStrategy
from areal_b200.api.cli_args import TrainEngineConfig
from areal_b200.infra.controller.train_controller import (TrainController, dispatch_batch, merge_outputs,
                                                           pad_batch_for_dispatch, strip_padding)
from areal_b200.infra.scheduler.local import LocalScheduler


def _batch(lens):
    L = max(lens)
    mask = torch.arange(L)[None, :] < torch.tensor(lens)[:, None]
    return dict(input_ids=(torch.arange(len(lens))[:, None] + 1).expand(-1, L) * mask, attention_mask=mask,
                rewards=torch.arange(len(lens)).float())


def test_dispatch_is_balanced_and_group_atomic_and_merge_inverts():
    lens = [10, 90, 20, 80, 30, 70, 40, 60]
    b = _batch(lens)
    parts, rows = dispatch_batch(b, 2, group_size=2)
    assert sorted(r for rr in rows for r in rr) == list(range(8))
    for rr in rows:
        assert len(rr) == 4 and all(rr[i] + 1 == rr[i + 1] for i in range(0, 4, 2))
    tok = [int(p["attention_mask"].sum()) for p in parts]
    assert abs(tok[0] - tok[1]) <= 40
    outs = [p["input_ids"].float() * 2 for p in parts]
    merged = merge_outputs(outs, rows)
    assert torch.equal(merged, b["input_ids"].float() * 2)
    st = merge_outputs([{"loss": 1.0, "n": 2.0}, {"loss": 3.0, "n": 4.0}], rows)
    assert st == {"loss": 2.0, "n": 3.0}


@pytest.mark.parametrize("n,dp,g,expect_pad", [(8, 4, 1, 0), (7, 4, 1, 1), (2, 4, 1, 2), (6, 4, 2, 2), (6, 3, 2, 0),
                                               (2, 3, 2, 4)])
def test_eval_batches_are_padded_with_weightless_samples(n, dp, g, expect_pad):
    b = _batch([5 + i for i in range(n)])
    b["loss_mask"] = b["attention_mask"].clone().int()
    b["images"] = [f"img{i}" for i in range(n)]
    b["meta"] = "shared"
    padded, n_pad = pad_batch_for_dispatch(b, dp, g)
    assert n_pad == expect_pad and padded["attention_mask"].shape[0] == n + n_pad
    if n_pad == 0:
        assert padded is b
        return
    assert torch.equal(padded["input_ids"][:n], b["input_ids"]) and padded["meta"] == "shared"
    assert padded["images"] == b["images"] + [None] * n_pad
    assert padded["attention_mask"][n:].sum(-1).tolist() == [1] * n_pad      # one-token sequences
    assert int(padded["loss_mask"][n:].sum()) == 0                            # no loss weight
    parts, rows = dispatch_batch(padded, dp, g)                               # now it divides
    assert len(parts) == dp
    merged = merge_outputs([p["input_ids"].float() for p in parts], rows)
    assert torch.equal(strip_padding(merged, n, n_pad), b["input_ids"].float())
    assert strip_padding({"x": merged, "s": 1.0}, n, n_pad)["x"].shape[0] == n
    with pytest.raises(AssertionError):
        dispatch_batch(b, dp, g)                                              # the unpadded batch does not


class _FakeAlloc:
    world_size = 2
    parallel = ParallelStrategy(data_parallel_size=2)


def test_train_controller_fanout(tmp_path):
    sched = LocalScheduler(gpu_devices=[], log_dir=str(tmp_path))
    cfg = TrainEngineConfig(backend="fsdp:d2")
    ctl = TrainController("tests.fake_engine.FakeTrainEngine", cfg, sched)
    # the fake engine has no process-group methods: wire the workers by hand
    from areal_b200.api.scheduler_api import Job
    import asyncio

    sched.create_workers(Job(replicas=2, role="actor"))
    ctl.workers = sched.get_workers("actor", timeout=60)
    ctl.role, ctl.alloc = "actor", _FakeAlloc()
    async def make():
        await asyncio.gather(*[sched.create_engine(w.id, "tests.fake_engine.FakeTrainEngine", scale=2.0,
                                                   engine_name="actor") for w in ctl.workers])

    asyncio.run(make())
    try:
        b = _batch([5, 9, 3, 7])
        out = ctl.forward_batch(b)
        assert torch.equal(out, b["input_ids"].float() * 2)
        st = ctl.train_batch(b, None, None)
        assert st["n"] == pytest.approx(6.0)  # 3 tensors x 2 rows on each rank (averaged over the two ranks)
        ctl.set_version(3)
        assert ctl.get_version() == 3 and sched.call_engine("actor/1", "get_version", "actor") == 3
        assert len(ctl._remote_shards) > 0
        ctl.clear_batches()
        assert ctl._remote_shards == []
    finally:
        ctl.destroy()
