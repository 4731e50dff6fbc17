"""Disaggregated rollout ↔ trainer plumbing inside one ``torch.distributed`` world.

Rollout ranks run a :class:`NativeRolloutEngine`; trainer ranks drive them
through :class:`RemoteRolloutClient`, which looks like an ``InferenceEngine`` to
the trainer. Per paired (rollout rank, trainer rank):

* trajectories travel rollout → trainer as pickled tensor dicts over a gloo
  group (a few MB per step);
* control messages (pause / resume+version / stop) travel trainer → rollout over
  a second gloo group, served by a control thread on the rollout rank;
* weights travel trainer → rollout **directly through peer memory**: every
  trainer rank copies its shard of the flat bf16 weights into the flat weight
  buffer of every rollout rank with one kernel over NVLink
  (``b200_push_all``). No rank-0 funnel, no per-tensor broadcast.

This replaces the reference's HTTP control plane plus NCCL broadcast from trainer
rank 0 to all inference ranks (areal/engine/fsdp_engine.py:1377-1597,
areal/infra/dist_rollout.py:29-148) and its redistribution of trajectories
across data-parallel ranks.
"""

from __future__ import annotations

import ctypes
import threading
import time
from typing import Any

import torch
import torch.distributed as dist

from ..api.engine_api import InferenceEngine
from ..ops import _lib
from ..parallel.symm_mem import open_ipc_handle
from ..utils import logging
from ..utils.data import concat_padded_tensors
from ..utils.seqpack import balanced_greedy_partition

logger = logging.getLogger("DistRollout")


class DisaggTopology:
    """Rank layout: ``[0, n_gen)`` rollout, ``[n_gen, n_gen + n_train)`` trainers. Rollout ranks are paired
    with the *heads* of the trainer's data-parallel replicas: under tensor / sequence / pipeline parallelism
    the ``replica_size`` ranks of a replica train one batch, which its first rank fetches and shares."""

    def __init__(self, n_gen: int, n_train: int, replica_size: int = 1, n_replicas: int | None = None):
        self.n_gen, self.n_train = n_gen, n_train
        self.world = dist.get_world_size()
        assert n_gen + n_train == self.world, f"allocation {n_gen}+{n_train} != world {self.world}"
        self.rank = dist.get_rank()
        self.gen_ranks = list(range(n_gen))
        self.train_ranks = list(range(n_gen, n_gen + n_train))
        self.is_rollout = self.rank < n_gen
        n_replicas = n_replicas if n_replicas is not None else max(n_train // max(replica_size, 1), 1)
        # tp is innermost, then sequence parallel, then data parallel, pipeline stages outermost: the head of
        # replica d is the rank at offset d * replica_size of the first stage
        self.train_heads = [self.train_ranks[d * replica_size] for d in range(n_replicas)]
        # gloo groups over the whole world: one for data, one for control
        self.data_group = dist.new_group(list(range(self.world)), backend="gloo")
        self.ctl_group = dist.new_group(list(range(self.world)), backend="gloo")
        self.all_cpu_group = dist.new_group(list(range(self.world)), backend="gloo")

    def trainers_of(self, gen_rank: int) -> list[int]:
        heads = self.train_heads
        return [t for i, t in enumerate(heads) if i % self.n_gen == gen_rank % self.n_gen] \
            if len(heads) >= self.n_gen else [heads[gen_rank % len(heads)]]

    def rollouts_of(self, train_rank: int) -> list[int]:
        return [g for g in self.gen_ranks if train_rank in self.trainers_of(g)]


def exchange_weight_buffers(topo: DisaggTopology, rollout_engine=None, device_index: int = 0) -> list[int]:
    """Collective over the world: rollout ranks export their flat weight buffer, trainer
    ranks map all of them. Returns the mapped pointers on trainer ranks ([] on rollout ranks).
    The rollout engine's parameter layout travels along (``topo.rollout_layout``): a model-parallel trainer
    needs it to re-shard on the way (``infra/weight_plan.py``)."""
    handle = None
    if topo.is_rollout:
        from .weight_plan import rollout_layout

        layout = rollout_layout(rollout_engine.flat) if topo.rank == topo.gen_ranks[0] else None
        handle = (rollout_engine.flat.param_buf.ipc_handle() if rollout_engine.flat.cuda else None,
                  rollout_engine.flat.numel, layout)
    handles: list[Any] = [None] * topo.world
    dist.all_gather_object(handles, handle, group=topo.all_cpu_group)
    topo.rollout_layout = handles[topo.gen_ranks[0]][2]
    if topo.is_rollout:
        return []
    if any(handles[g][0] is None for g in topo.gen_ranks):
        return []  # CPU ranks: weights travel over gloo instead (see receive_weights)
    return [open_ipc_handle(handles[g][0], device_index) for g in topo.gen_ranks]


class RolloutServer:
    """Runs on a rollout rank: produces batches for its trainer(s) and obeys control messages."""

    def __init__(self, topo: DisaggTopology, engine):
        self.topo, self.engine = topo, engine
        self.trainers = topo.trainers_of(topo.rank)
        self._stop = threading.Event()
        self._eval: tuple | None = None  # (items of this rank, workflow, workflow kwargs)
        self._ctl_thread = threading.Thread(target=self._control_loop, name="rollout-ctl", daemon=True)
        self._ctl_thread.start()

    def set_eval(self, items: list, workflow, workflow_kwargs=None):
        """What an ``("eval",)`` command runs: this rank's share of the validation set through ``workflow``."""
        self._eval = (list(items), workflow, workflow_kwargs)

    def _run_eval(self) -> tuple[float, int]:
        """Sum of rewards and number of scored samples. The episodes run on a private event loop of the control
        thread, straight against the engine (not through the workflow executor, whose result queue belongs to
        the training loop on the main thread); generation for training goes on meanwhile."""
        if self._eval is None or not self._eval[0]:
            return 0.0, 0
        import asyncio

        from .workflow_executor import resolve_workflow

        items, workflow, kwargs = self._eval
        wf = resolve_workflow(workflow, kwargs)

        async def run_all():
            return await asyncio.gather(*[wf.arun_episode(self.engine, dict(it)) for it in items],
                                        return_exceptions=True)

        total, n = 0.0, 0
        for out in asyncio.run(run_all()):
            if out is None or isinstance(out, BaseException):
                continue
            for traj in (out if isinstance(out, list) else [out]):
                r = traj["rewards"].float()
                total, n = total + float(r.sum()), n + int(r.numel())
        return total, n

    def _control_loop(self):
        lead = self.trainers[0]
        while not self._stop.is_set():
            msg = [None]
            dist.recv_object_list(msg, src=lead, group=self.topo.ctl_group)
            cmd = msg[0]
            if cmd[0] == "pause":
                self.engine.pause_generation()
                dist.send_object_list([("ack", time.time())], dst=lead, group=self.topo.ctl_group)
            elif cmd[0] == "weights":
                # CPU fallback: every trainer rank sends its shard of the flat weights over gloo
                flat = self.engine.flat.flat
                shard = cmd[1]
                for i, t in enumerate(self.topo.train_ranks):
                    buf = torch.empty(shard, dtype=flat.dtype)
                    dist.recv(buf, src=t, group=self.topo.ctl_group)
                    n = min(shard, flat.numel() - i * shard)
                    if n > 0:
                        flat[i * shard: i * shard + n].copy_(buf[:n])
            elif cmd[0] == "resume":
                if cmd[1] is not None:
                    self.engine.set_version(cmd[1])
                self.engine.continue_generation()
            elif cmd[0] == "eval":
                dist.send_object_list([("eval_result",) + self._run_eval()], dst=lead, group=self.topo.ctl_group)
            elif cmd[0] == "stop":
                self._stop.set()
                return

    def serve(self, dataloader, workflow, workflow_kwargs=None, group_size: int = 1, n_steps: int | None = None):
        """Produces ``n_steps`` batches (forever if ``None``) and ships each, split evenly by token
        count, to the paired trainer ranks."""
        step = 0
        while not self._stop.is_set() and (n_steps is None or step < n_steps):
            batch = self.engine.prepare_batch(dataloader, workflow, workflow_kwargs, group_size=group_size)
            parts = split_batch_by_tokens(batch, len(self.trainers), group_size)
            stats = self.engine.export_stats() if hasattr(self.engine, "export_stats") else {}
            for t, part in zip(self.trainers, parts):
                # the engine's counters ride along, so the trainer side can report per-role rates
                dist.send_object_list([part, stats], dst=t, group=self.topo.data_group)
            step += 1

    def wait_stop(self, timeout: float | None = None):
        self._ctl_thread.join(timeout)


def split_batch_by_tokens(batch: dict[str, Any], k: int, group_size: int = 1) -> list[dict[str, Any]]:
    """Splits a padded batch into ``k`` parts with balanced token counts, keeping each
    group of ``group_size`` consecutive samples together."""
    if k == 1:
        return [batch]
    B = batch["attention_mask"].shape[0]
    lens = batch["attention_mask"].sum(-1).tolist()
    g = max(group_size, 1)
    units = [sum(lens[i:i + g]) for i in range(0, B, g)]
    parts = balanced_greedy_partition(units, k, equal_size=True)
    out = []
    for p in parts:
        rows = torch.tensor([u * g + j for u in sorted(p) for j in range(g)], dtype=torch.long)
        out.append({key: (v[rows] if torch.is_tensor(v) and v.dim() >= 1 and v.shape[0] == B else v)
                    for key, v in batch.items()})
    return out


class RemoteRolloutClient(InferenceEngine):
    """Trainer-side handle of the paired rollout rank(s)."""

    def __init__(self, topo: DisaggTopology, weight_ptrs: list[int], train_cpu_group=None):
        self.topo = topo
        self.rollouts = topo.rollouts_of(topo.rank)
        # the lead trainer of a rollout rank is the one that sends it control messages
        self.led = [g for g in self.rollouts if topo.trainers_of(g)[0] == topo.rank]
        self.weight_ptrs = weight_ptrs
        self.train_cpu_group = train_cpu_group
        self._version = 0
        self._table = (ctypes.c_void_p * max(len(weight_ptrs), 1))(*weight_ptrs) if weight_ptrs else None
        self.last_pause_latency = 0.0
        self.rollout_stats: dict[int, dict[str, float]] = {}  # rollout rank -> its engine's latest counters
        self._pusher = None

    def prepare_batch(self, dataloader=None, workflow=None, workflow_kwargs=None, should_accept_fn=None,
                      group_size=1, dynamic_bs=False):
        parts = []
        for g in self.rollouts:
            msg = [None, None]
            dist.recv_object_list(msg, src=g, group=self.topo.data_group)
            parts.append(msg[0])
            self.rollout_stats[g] = msg[1] or {}
        return parts[0] if len(parts) == 1 else concat_padded_tensors(parts)

    rollout_batch = prepare_batch

    def pause_generation(self):
        t0 = time.perf_counter()
        for g in self.led:
            dist.send_object_list([("pause",)], dst=g, group=self.topo.ctl_group)
        for g in self.led:
            msg = [None]
            dist.recv_object_list(msg, src=g, group=self.topo.ctl_group)
        if self.train_cpu_group is not None:
            dist.barrier(group=self.train_cpu_group)  # every rollout rank has paused
        self.last_pause_latency = time.perf_counter() - t0

    def continue_generation(self, version: int | None = None):
        if self.train_cpu_group is not None:
            dist.barrier(group=self.train_cpu_group)  # every trainer's shard has landed
        for g in self.led:
            dist.send_object_list([("resume", version if version is not None else self._version)],
                                  dst=g, group=self.topo.ctl_group)

    def receive_weights(self, trainer, version: int | None = None):
        """Each trainer rank writes its shard of the flat bf16 weights into every rollout
        rank's weight buffer (peer stores over NVLink), then synchronises its stream."""
        f = getattr(trainer, "weight_flat", trainer.flat)
        itemsize = f.flat.element_size()
        shard = f.flat[f.shard_offset: f.shard_offset + f.shard_numel]
        ps = getattr(trainer, "parallel", None)
        if ps is not None and ps.tp_size * ps.pp_size * ps.ep_size > 1:
            # the trainer holds shards (slices of fused projections, a stage's blocks, some experts): each
            # rank pushes its share of a re-sharding plan straight into every rollout buffer
            if not self.weight_ptrs:
                raise NotImplementedError("re-sharding weight push needs CUDA peer memory")
            if self._pusher is None:
                from .weight_plan import WeightPusher

                self._pusher = WeightPusher(trainer, self.weight_ptrs, self.topo.rollout_layout)
            self._pusher.push()
            torch.cuda.current_stream().synchronize()
            if version is not None:
                self._version = version
            return
        if not self.weight_ptrs:
            for g in self.led:
                dist.send_object_list([("weights", f.shard_numel)], dst=g, group=self.topo.ctl_group)
            if self.train_cpu_group is not None:
                dist.barrier(group=self.train_cpu_group)
            for g in self.topo.gen_ranks:
                dist.send(shard.contiguous(), dst=g, group=self.topo.ctl_group)
            if version is not None:
                self._version = version
            return
        lib = _lib.kernels()
        rc = lib.b200_push_all(self._table, ctypes.c_int(len(self.weight_ptrs)), _lib.ptr(shard),
                               ctypes.c_longlong(f.shard_numel * itemsize),
                               ctypes.c_longlong(f.shard_offset * itemsize), _lib.stream_ptr())
        _lib.check(rc, "b200_push_all")
        _lib.count_launch()
        torch.cuda.current_stream().synchronize()
        if version is not None:
            self._version = version

    def evaluate(self) -> tuple[float, int]:
        """Asks the led rollout ranks to run their share of the validation set; returns the sum of rewards and
        the sample count over all rollout ranks (reduced over the trainer ranks when they share a group)."""
        for g in self.led:
            dist.send_object_list([("eval",)], dst=g, group=self.topo.ctl_group)
        total, n = 0.0, 0
        for g in self.led:
            msg = [None]
            dist.recv_object_list(msg, src=g, group=self.topo.ctl_group)
            total, n = total + float(msg[0][1]), n + int(msg[0][2])
        if self.train_cpu_group is not None:
            acc = torch.tensor([total, float(n)], dtype=torch.float64)
            dist.all_reduce(acc, group=self.train_cpu_group)
            total, n = float(acc[0]), int(acc[1])
        return total, n

    def set_version(self, version: int):
        self._version = version

    def get_version(self) -> int:
        return self._version

    def pause(self):
        pass

    def resume(self):
        pass

    def stop(self):
        for g in self.led:
            dist.send_object_list([("stop",)], dst=g, group=self.topo.ctl_group)

    def export_stats(self) -> dict[str, float]:
        return {"rollout/pause_latency": self.last_pause_latency}


# --------------------------------------------------------------------------- rollout under a model-parallel trainer
class RedistributedData:
    """What :func:`redistribute_trajectories` returns: every rank's share (``all_data``), this rank's own
    (``data``), the row indices of the pooled batch that went to each rank (``group_indices``) and this rank's
    index."""

    def __init__(self, all_data: list[dict[str, Any]], data: dict[str, Any], rank: int, group_indices: list[list[int]]):
        self.all_data, self.data, self.rank, self.group_indices = all_data, data, rank, group_indices


def redistribute_trajectories(batch: dict[str, Any] | None, group=None, granularity: int = 1,
                              algorithm: str = "greedy") -> RedistributedData:
    """Pools the batches that the data-parallel heads rolled out and deals them out again so that every rank trains
    on about the same number of tokens: sequence lengths of asynchronous rollouts vary a lot, and the step takes as
    long as the most loaded rank. ``granularity`` consecutive samples (a sample group) stay on one rank.
    ``algorithm``: ``greedy`` (largest first into the lightest rank, equal sample counts) or ``kk``
    (Karmarkar-Karp). ``group``: the data-parallel group (``None`` with one rank: the batch comes back as it is)."""
    from ..utils.data import all_gather_tensor_container
    from ..utils.seqpack import kk_allocate

    world = dist.get_world_size(group) if (dist.is_initialized() and group is not None) else 1
    rank = dist.get_rank(group) if world > 1 else 0
    pooled = all_gather_tensor_container(batch, group) if world > 1 else [batch]
    pooled = [b for b in pooled if b]
    if not pooled:
        return RedistributedData([], {}, rank, [])
    whole = pooled[0] if len(pooled) == 1 else concat_padded_tensors(pooled)
    if world == 1:
        B = whole["attention_mask"].shape[0]
        return RedistributedData([whole], whole, 0, [list(range(B))])
    B = whole["attention_mask"].shape[0]
    g = max(granularity, 1)
    assert B % g == 0 and (B // g) >= world, f"{B} samples in groups of {g} cannot feed {world} ranks"
    lens = whole["attention_mask"].sum(-1).tolist()
    units = [int(sum(lens[i:i + g])) for i in range(0, B, g)]
    parts = kk_allocate(units, world, equal_size=True) if algorithm == "kk" else \
        balanced_greedy_partition(units, world, equal_size=(len(units) % world == 0))
    indices = [[u * g + j for u in sorted(p) for j in range(g)] for p in parts]
    shares = []
    for rows in indices:
        idx = torch.tensor(rows, dtype=torch.long)
        shares.append({k: (v[idx] if torch.is_tensor(v) and v.dim() >= 1 and v.shape[0] == B else
                           ([v[i] for i in rows] if isinstance(v, list) and len(v) == B else v))
                       for k, v in whole.items()})
    return RedistributedData(shares, shares[rank], rank, indices)


class DistRolloutCoordinator:
    """Rollout for a trainer with model parallelism: only the data-parallel heads talk to the inference engine, the
    trajectories are re-balanced over the data-parallel ranks by token count, and every rank of a replica
    (tensor / sequence / pipeline peers) receives its head's share.
    Reference: areal/infra/dist_rollout.py (DistRolloutCoordinator :97, redistribute_trajectories)."""

    def __init__(self, rollout_engine: InferenceEngine, train_engine):
        self.rollout_engine, self.train_engine = rollout_engine, train_engine

    def _finish(self, batch, granularity: int):
        from ..utils.data import broadcast_tensor_container

        te = self.train_engine
        if te.is_data_parallel_head():
            dp_group = te.data_parallel_group if te.data_parallel_world_size > 1 else None
            batch = redistribute_trajectories(batch, dp_group, granularity).data
        group = te.context_and_model_parallel_group
        if group is None:
            return batch
        return broadcast_tensor_container(batch, src_rank=te.current_data_parallel_head(), group=group)

    def rollout_batch(self, data, workflow=None, workflow_kwargs=None, group_size: int = 1):
        batch = None
        if self.train_engine.is_data_parallel_head():
            batch = self.rollout_engine.rollout_batch(data, workflow, workflow_kwargs, group_size=group_size)
        return self._finish(batch, group_size)

    def prepare_batch(self, dataloader, workflow=None, workflow_kwargs=None, should_accept_fn=None,
                      group_size: int = 1, dynamic_bs: bool = False):
        batch = None
        if self.train_engine.is_data_parallel_head():
            batch = self.rollout_engine.prepare_batch(dataloader, workflow, workflow_kwargs, should_accept_fn,
                                                      group_size=group_size, dynamic_bs=dynamic_bs)
        return self._finish(batch, group_size)
