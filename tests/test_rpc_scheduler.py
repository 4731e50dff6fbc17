"""Serialization envelopes, RTensor handles, the RPC server and the local scheduler
(real subprocess workers on localhost with a CPU fake engine)."""
import asyncio
import dataclasses
import enum

import numpy as np
import pytest
import torch

from areal_b200.api.cli_args import GenerationHyperparameters, SchedulingSpec
from areal_b200.api.io_struct import ModelRequest
from areal_b200.api.scheduler_api import Job
from areal_b200.infra.rpc import rtensor
from areal_b200.infra.rpc.serialization import deserialize_value, serialize_value
from areal_b200.infra.scheduler.exceptions import (EngineCallError, WorkerCreationError, WorkerFailedError,
                                                   WorkerNotFoundError)
from areal_b200.infra.scheduler.local import LocalScheduler


class Color(enum.Enum):
    RED = "r"


def test_serialization_roundtrip():
    v = {"t": torch.arange(6).view(2, 3), "bf": torch.randn(3).bfloat16(), "np": np.ones((2, 2), dtype=np.float32),
         "tup": (1, "a", 2.5), "set": {1, 2}, "b": b"xyz", "e": Color.RED, "n": None,
         "dc": ModelRequest(input_ids=[1, 2], gconfig=GenerationHyperparameters(max_new_tokens=7)), 3: "int-key"}
    out = deserialize_value(serialize_value(v))
    assert torch.equal(out["t"], v["t"]) and torch.equal(out["bf"], v["bf"]) and out["bf"].dtype == torch.bfloat16
    assert np.array_equal(out["np"], v["np"]) and out["tup"] == (1, "a", 2.5) and out["set"] == {1, 2}
    assert out["b"] == b"xyz" and out["e"] is Color.RED and out["n"] is None and out[3] == "int-key"
    assert out["dc"].input_ids == [1, 2] and out["dc"].gconfig.max_new_tokens == 7
    with pytest.raises(TypeError):
        serialize_value(object())


def test_rtensor_local_roundtrip():
    batch = {"a": torch.randn(4, 3), "meta": {"ids": [torch.arange(3)], "k": 5}}
    h = rtensor.remotize(batch)
    assert isinstance(h["a"], rtensor.RTensor) and h["a"].shape == (4, 3) and h["meta"]["k"] == 5
    assert h["a"].meta.device.type == "meta"
    wire = deserialize_value(serialize_value(h))
    back = rtensor.localize(wire)
    assert torch.equal(back["a"], batch["a"]) and torch.equal(back["meta"]["ids"][0], torch.arange(3))
    ids = [s for _, s in rtensor.collect_shard_ids(h)]
    assert len(ids) == 2
    rtensor.LOCAL_STORE.delete(ids)
    with pytest.raises(KeyError):
        rtensor.localize(h)


def test_rtensor_shards_on_several_owners_backend_buffer_and_removal():
    """A handle over the rows of two workers: localising fetches each owner once (all its shards in one request),
    pads the ragged sequence dimension and concatenates; a second localise is served from the fetch buffer."""
    mem = rtensor.MemoryBackend()
    prev = rtensor.set_backend(mem)
    rtensor.clear_fetch_buffer()
    try:
        a1, a2, b1 = torch.ones(2, 3), torch.full((1, 3), 2.0), torch.full((2, 5), 3.0)
        s1, s2 = rtensor.store(a1, "w0:1"), rtensor.store(a2, "w0:1")
        s3 = rtensor.store(b1, "w1:1")
        assert (s1.addr, s1.rows) == ("w0:1", 2) and len(mem.stores["w0:1"]) == 2
        parts = [rtensor.RTensor(s.shard_id, s.addr, tuple(t.shape), "float32") for s, t in ((s1, a1), (s2, a2), (s3, b1))]
        h = rtensor.RTensor.cat(parts)
        assert h.shape == (5, 5) and len(h.shard_infos()) == 3
        wire = deserialize_value(serialize_value({"x": h}))["x"]
        assert [s.shard_id for s in wire.shard_infos()] == [s1.shard_id, s2.shard_id, s3.shard_id]
        before = rtensor.fetch_buffer_stats()
        full = wire.to_local()
        assert full.shape == (5, 5) and full[:2, :3].eq(1).all() and full[:3, 3:].eq(0).all() and full[3:].eq(3).all()
        assert mem.fetches == 2                                       # one request per owner, not per shard
        again = rtensor.localize({"x": h})["x"]
        st = rtensor.fetch_buffer_stats()
        assert torch.equal(again, full) and mem.fetches == 2 and st["hits"] - before["hits"] == 3 and st["entries"] == 3
        assert sorted(rtensor.flatten_shard_ids({"x": h, "y": [parts[0]]})) == sorted([s1.shard_id, s2.shard_id, s3.shard_id, s1.shard_id])
        rtensor.remove([s1, s2])
        assert len(mem.stores["w0:1"]) == 0 and rtensor.fetch_buffer_stats()["entries"] == 1
        with pytest.raises(KeyError):
            wire.to_local()
        local = rtensor.store(torch.zeros(4))
        assert rtensor.storage_stats()["entries"] >= 1 and rtensor.fetch([local])[0].shape == (4,)
        rtensor.remove([local])
        with pytest.raises(ValueError):
            rtensor.RTensor.cat([])
        with pytest.raises(ImportError):
            rtensor.RayRTensorBackend()
    finally:
        rtensor.set_backend(prev)
        rtensor.clear_fetch_buffer()


@pytest.fixture
def sched(tmp_path):
    s = LocalScheduler(gpu_devices=[0, 1], log_dir=str(tmp_path), startup_timeout=60)
    yield s
    s.delete_workers()


def test_local_scheduler_lifecycle_and_engine_calls(sched):
    ids = sched.create_workers(Job(replicas=2, tasks=[SchedulingSpec(gpu=1)], role="actor"))
    assert ids == ["actor/0", "actor/1"]
    workers = sched.get_workers("actor", timeout=60)
    assert len(workers) == 2 and sched._by_id["actor/0"].gpus != sched._by_id["actor/1"].gpus
    with pytest.raises(WorkerCreationError):
        sched.create_workers(Job(replicas=1, role="actor"))
    # colocated role shares the GPUs of its target
    from areal_b200.api.cli_args import SchedulingStrategy

    sched.create_workers(Job(replicas=2, role="ref", scheduling_strategy=SchedulingStrategy("colocation", "actor")))
    assert sched._by_id["ref/1"].gpus == sched._by_id["actor/1"].gpus
    sched.get_workers("ref", timeout=60)
    asyncio.run(sched.create_engine("actor/0", "tests.fake_engine.FakeTrainEngine", scale=3.0))
    out = sched.call_engine("actor/0", "train_batch", None, {"x": torch.ones(2, 2)})
    assert out["sum"] == pytest.approx(12.0) and out["calls"] == 1
    out = asyncio.run(sched.async_call_engine("actor/0", "train_batch", None, {"x": torch.ones(1)}))
    assert out["calls"] == 2
    # tensors can stay on the worker and travel as handles
    h = sched.call_engine("actor/0", "make_batch", None, 5, return_rtensor=True)
    assert isinstance(h["ids"], rtensor.RTensor) and h["ids"].addr is not None
    assert torch.equal(h["ids"].to_local(), torch.arange(5))
    assert sched.call_engine("actor/0", "consume", None, h) == 10
    with pytest.raises(EngineCallError):
        sched.call_engine("actor/0", "explode", None)
    with pytest.raises(EngineCallError):
        sched.call_engine("actor/1", "train_batch", None, {})  # no engine on this worker
    with pytest.raises(WorkerNotFoundError):
        sched.call_engine("nobody/0", "x", None)
    sched.delete_workers("ref")
    with pytest.raises(WorkerNotFoundError):
        sched.get_workers("ref")


def test_dead_worker_is_detected(sched):
    sched.create_workers(Job(replicas=1, role="w"))
    sched.get_workers("w", timeout=60)
    asyncio.run(sched.create_engine("w/0", "tests.fake_engine.FakeTrainEngine"))
    sched._by_id["w/0"].process.kill()
    sched._by_id["w/0"].process.wait()
    with pytest.raises(WorkerFailedError):
        sched.call_engine("w/0", "train_batch", None, {"x": torch.ones(1)})


def test_serialization_of_images_processor_outputs_and_tokenizers(monkeypatch):
    """What a vision-language trajectory carries across RPC: PIL images, a processor's mapping-type output, and
    tokenizers / processors by the path they were loaded from."""
    import collections

    from PIL import Image

    img = Image.fromarray((np.arange(12 * 10 * 3) % 255).astype("uint8").reshape(12, 10, 3))
    feat = collections.UserDict(pixel_values=torch.ones(4, 6), image_grid_thw=torch.tensor([[1, 2, 2]]))
    out = deserialize_value(serialize_value({"img": img, "mm": [feat]}))
    assert out["img"].size == (10, 12) and np.array_equal(np.asarray(out["img"]), np.asarray(img))
    assert isinstance(out["mm"][0], dict) and torch.equal(out["mm"][0]["pixel_values"], feat["pixel_values"])

    class Tok:
        name_or_path = "/models/some-model"

        def encode(self, text):
            return []

    env = serialize_value({"tok": Tok()})
    assert env["tok"] == {"__type__": "tokenizer", "path": "/models/some-model"}
    import transformers

    loaded = []
    monkeypatch.setattr(transformers.AutoTokenizer, "from_pretrained", classmethod(lambda cls, p: loaded.append(p) or "tok"))
    assert deserialize_value(env)["tok"] == "tok" and loaded == ["/models/some-model"]
    Tok.name_or_path = ""
    with pytest.raises(TypeError):
        serialize_value(Tok())
