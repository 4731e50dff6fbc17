"""Single-controller stand-in for a train engine.

The controller process owns no model. ``initialize`` asks the scheduler for one
worker per rank, wires the torch.distributed environment, creates the engine in
every worker and initialises it. Every engine method is then a fan-out RPC:
batches are split across data-parallel heads (token-balanced, GRPO groups kept
together), shipped as :class:`RTensor` handles, executed concurrently, and the
per-rank results merged in the original sample order
(role of areal/infra/controller/train_controller.py:76-868 in the reference).
"""

from __future__ import annotations

import asyncio
import uuid
from typing import Any

import requests
import torch

from ...api.alloc_mode import ModelAllocation
from ...api.cli_args import SchedulingSpec, TrainEngineConfig
from ...api.io_struct import FinetuneSpec, SaveLoadMeta, WeightUpdateMeta
from ...api.scheduler_api import Job, Scheduler, Worker
from ...utils import logging
from ...utils.seqpack import balanced_greedy_partition
from ..rpc.rpc_server import find_free_ports
from ..rpc.rtensor import RTensor
from ..rpc.serialization import serialize_value

logger = logging.getLogger("TrainController")


def dispatch_batch(batch: dict[str, Any], n_parts: int, group_size: int = 1) -> tuple[list[dict[str, Any]], list[list[int]]]:
    """Token-balanced split into ``n_parts`` with equal sample counts; groups of ``group_size``
    consecutive samples stay on one rank. Returns the parts and their original row indices."""
    B = batch["attention_mask"].shape[0]
    g = max(group_size, 1)
    assert B % g == 0 and (B // g) % n_parts == 0, f"batch {B} (groups of {g}) does not split over {n_parts} ranks"
    lens = batch["attention_mask"].sum(-1).tolist()
    units = [sum(lens[i:i + g]) for i in range(0, B, g)]
    groups = balanced_greedy_partition(units, n_parts, equal_size=True)
    parts, rows_all = [], []
    for grp in groups:
        rows = [u * g + j for u in sorted(grp) for j in range(g)]
        idx = torch.tensor(rows, dtype=torch.long)
        parts.append({k: (v[idx] if torch.is_tensor(v) and v.dim() >= 1 and v.shape[0] == B else v)
                      for k, v in batch.items()})
        rows_all.append(rows)
    return parts, rows_all


def pad_batch_for_dispatch(batch: dict[str, Any], n_parts: int, group_size: int = 1) -> tuple[dict[str, Any], int]:
    """Evaluation and inference batches need not divide over the data-parallel ranks (the tail of a validation
    set, fewer prompts than ranks): appends dummy samples up to the next multiple of ``n_parts`` groups and
    returns how many rows were added. A dummy sample is a one-token sequence with an all-zero ``loss_mask``, so
    it carries no loss weight and every per-sample tensor stays aligned with its row."""
    B = batch["attention_mask"].shape[0]
    g = max(group_size, 1)
    assert B % g == 0, f"batch {B} is not a whole number of groups of {g}"
    n_pad = ((-(B // g)) % n_parts) * g
    if n_pad == 0:
        return batch, 0
    out = {}
    for k, v in batch.items():
        if torch.is_tensor(v) and v.dim() >= 1 and v.shape[0] == B:
            pad = torch.zeros((n_pad,) + tuple(v.shape[1:]), dtype=v.dtype)
            if k == "attention_mask":
                pad[:, 0] = 1
            out[k] = torch.cat([v, pad])
        elif isinstance(v, list) and len(v) == B:
            out[k] = list(v) + [None] * n_pad  # per-sample payloads (images): dummies have none
        else:
            out[k] = v
    return out, n_pad


def strip_padding(merged: Any, n_real: int, n_pad: int) -> Any:
    """Drops the rows that :func:`pad_batch_for_dispatch` appended from a merged per-sample result."""
    if n_pad == 0:
        return merged
    if torch.is_tensor(merged) and merged.dim() >= 1 and merged.shape[0] == n_real + n_pad:
        return merged[:n_real]
    if isinstance(merged, dict):
        return {k: strip_padding(v, n_real, n_pad) for k, v in merged.items()}
    return merged


def merge_outputs(outs: list[Any], rows_all: list[list[int]]) -> Any:
    """Inverse of :func:`dispatch_batch` for per-sample tensors; dict stats are averaged."""
    first = outs[0]
    if torch.is_tensor(first):
        B = sum(len(r) for r in rows_all)
        L = max(o.shape[1] for o in outs) if first.dim() >= 2 else None
        shape = (B, L) + tuple(first.shape[2:]) if L is not None else (B,) + tuple(first.shape[1:])
        merged = torch.zeros(shape, dtype=first.dtype)
        for o, rows in zip(outs, rows_all):
            idx = torch.tensor(rows, dtype=torch.long)
            if L is not None:
                merged[idx, : o.shape[1]] = o
            else:
                merged[idx] = o
        return merged
    if isinstance(first, dict) and any(torch.is_tensor(v) for v in first.values()):
        # a batch: per-sample tensors are merged back in the original order, everything else is taken from the
        # first rank
        n_rows = [len(r) for r in rows_all]
        out = {}
        for k, v in first.items():
            if torch.is_tensor(v) and v.dim() >= 1 and all(torch.is_tensor(o[k]) and o[k].shape[0] == n
                                                           for o, n in zip(outs, n_rows)):
                out[k] = merge_outputs([o[k] for o in outs], rows_all)
            else:
                out[k] = v
        return out
    if isinstance(first, dict):
        keys = first.keys()
        return {k: (sum(float(o[k]) for o in outs) / len(outs)) if isinstance(first[k], (int, float)) else first[k]
                for k in keys}
    if isinstance(first, list) and first and isinstance(first[0], dict):
        return [merge_outputs([o[i] for o in outs], rows_all) for i in range(len(first))]
    return first


class TrainController:
    def __init__(self, engine: str | type, config: TrainEngineConfig, scheduler: Scheduler):
        self.engine_path = engine if isinstance(engine, str) else f"{engine.__module__}.{engine.__qualname__}"
        self.config = config
        self.scheduler = scheduler
        self.workers: list[Worker] = []
        self.role = "default"
        self.alloc: ModelAllocation | None = None
        self._version = 0
        self.group_size = 1
        self._remote_shards: list[tuple[str, str]] = []

    # ------------------------------------------------------------------- setup
    def initialize(self, role: str = "actor", alloc_mode: ModelAllocation | None = None,
                   ft_spec: FinetuneSpec | None = None, group_size: int = 1, **kwargs):
        self.role = role
        self.group_size = group_size
        self.alloc = alloc_mode or ModelAllocation.from_str(self.config.backend)
        world = self.alloc.world_size
        specs = list(self.config.scheduling_spec) or [SchedulingSpec()]
        job = Job(replicas=world, tasks=[specs[0]], scheduling_strategy=self.config.scheduling_strategy, role=role)
        self.scheduler.create_workers(job)
        self.workers = self.scheduler.get_workers(role, timeout=self.config.setup_timeout)
        port = find_free_ports(1)[0]

        async def setup():
            await asyncio.gather(*[
                self.scheduler.set_worker_env(w.id, dict(RANK=str(i), WORLD_SIZE=str(world), LOCAL_RANK="0",
                                                         MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port)))
                for i, w in enumerate(self.workers)])
            await asyncio.gather(*[self.scheduler.create_engine(w.id, self.engine_path, self.config,
                                                                engine_name=role) for w in self.workers])
            await self._call_all("create_process_group", self.alloc.parallel)
            await self._call_all("initialize", None, ft_spec, **kwargs)

        asyncio.run(setup())
        return self

    def destroy(self):
        try:
            self.scheduler.delete_workers(self.role)
        except Exception as e:
            logger.warning(f"could not delete workers of {self.role}: {e}")

    # ------------------------------------------------------------------ calls
    async def _call_all(self, method: str, *args, per_worker_args: list[tuple] | None = None, **kwargs) -> list[Any]:
        coros = []
        for i, w in enumerate(self.workers):
            a = per_worker_args[i] if per_worker_args is not None else args
            coros.append(self.scheduler.async_call_engine(w.id, method, self.role, *a, **kwargs))
        return await asyncio.gather(*coros)

    def _custom_function_call(self, method: str, *args, **kwargs):
        return asyncio.run(self._call_all(method, *args, **kwargs))[0]

    def _ship(self, worker: Worker, part: dict[str, Any]) -> dict[str, Any]:
        """Uploads the tensors of ``part`` into ``worker``'s shard store; returns handles."""
        addr = f"{worker.ip}:{worker.worker_ports[0]}"
        out = {}
        for k, v in part.items():
            if torch.is_tensor(v):
                sid = uuid.uuid4().hex
                r = requests.put(f"http://{addr}/data/{sid}", json=serialize_value(v), timeout=600)
                r.raise_for_status()
                out[k] = RTensor(sid, addr, tuple(v.shape), str(v.dtype).replace("torch.", ""))
                self._remote_shards.append((addr, sid))
            else:
                out[k] = v
        return out

    def _data_call(self, method: str, batch: dict[str, Any], *args, pad: bool = False, **kwargs):
        dp = self.alloc.parallel.dp_size
        n_real, n_pad = batch["attention_mask"].shape[0], 0
        if pad:
            batch, n_pad = pad_batch_for_dispatch(batch, dp, self.group_size)
        parts, rows = dispatch_batch(batch, dp, self.group_size)
        # every rank of a data-parallel group receives its head's part
        per_rank = len(self.workers) // dp
        handles = []
        for i, w in enumerate(self.workers):
            handles.append((self._ship(w, parts[i // per_rank]),) + args)
        outs = asyncio.run(self._call_all(method, per_worker_args=handles, **kwargs))
        heads = [outs[i * per_rank] for i in range(dp)]
        return strip_padding(merge_outputs(heads, rows), n_real, n_pad)

    # ------------------------------------------------------------- engine API
    def train_batch(self, input_: dict[str, Any], loss_fn, loss_weight_fn):
        return self._data_call("train_batch", input_, loss_fn, loss_weight_fn)

    def forward_batch(self, input_: dict[str, Any], *args, **kwargs):
        return self._data_call("forward_batch", input_, *args, pad=True, **kwargs)

    def eval_batch(self, input_: dict[str, Any], loss_fn, loss_weight_fn):
        return self._data_call("eval_batch", input_, loss_fn, loss_weight_fn, pad=True)

    # algorithm methods of an actor / critic engine created in the workers (``trainer.ppo.actor.PPOActorEngine``)
    def compute_logp(self, input_: dict[str, Any], *args, **kwargs):
        return self._data_call("compute_logp", input_, *args, **kwargs)

    def compute_values(self, input_: dict[str, Any], *args, **kwargs):
        return self._data_call("compute_values", input_, *args, **kwargs)

    def compute_advantages(self, input_: dict[str, Any], *args, **kwargs):
        return self._data_call("compute_advantages", input_, *args, **kwargs)

    def ppo_update(self, input_: dict[str, Any], *args, **kwargs):
        return self._data_call("ppo_update", input_, *args, **kwargs)

    def train(self, mode: bool = True):
        self._custom_function_call("train", mode)
        return self

    def eval(self):
        return self.train(False)

    def set_version(self, version: int):
        self._version = version
        self._custom_function_call("set_version", version)

    def get_version(self) -> int:
        return self._version

    def save(self, meta: SaveLoadMeta):
        self._custom_function_call("save", meta)

    def load(self, meta: SaveLoadMeta):
        self._custom_function_call("load", meta)

    def update_weights(self, meta: WeightUpdateMeta):
        self._custom_function_call("update_weights", meta)

    def export_stats(self) -> dict[str, float]:
        return self._custom_function_call("export_stats")

    def clear_batches(self, *args):
        """Frees the shards uploaded for previous calls."""
        by_addr: dict[str, list[str]] = {}
        for addr, sid in self._remote_shards:
            by_addr.setdefault(addr, []).append(sid)
        for addr, ids in by_addr.items():
            try:
                requests.post(f"http://{addr}/data/clear", json={"shard_ids": ids}, timeout=60)
            except requests.RequestException as e:
                logger.warning(f"could not clear shards on {addr}: {e}")
        self._remote_shards.clear()

    def __getattr__(self, name: str):
        # any other engine method is a plain fan-out call
        if name.startswith("_"):
            raise AttributeError(name)
        return lambda *a, **k: self._custom_function_call(name, *a, **k)
