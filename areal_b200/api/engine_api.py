"""Engine contracts.

``TrainEngine`` is the data-plane interface of every training back end and
``InferenceEngine`` the interface of the rollout side; trainers, controllers and
workflows are written against these (method set as in
areal/api/engine_api.py:32-1008 of the reference).
"""

from __future__ import annotations

import abc
from concurrent.futures import Future
from typing import TYPE_CHECKING, Any, Callable

import torch

from .io_struct import (FinetuneSpec, ModelRequest, ModelResponse, ParamSpec, SaveLoadMeta,
                        WeightUpdateMeta)

if TYPE_CHECKING:
    from .workflow_api import RolloutWorkflow


class TrainEngine(abc.ABC):
    def create_process_group(self, parallel_strategy=None):
        raise NotImplementedError

    def initialize(self, addr: str | None = None, ft_spec: FinetuneSpec | None = None, *args, **kwargs):
        raise NotImplementedError

    @property
    def data_parallel_group(self):
        raise NotImplementedError

    @property
    def data_parallel_rank(self) -> int:
        raise NotImplementedError

    @property
    def data_parallel_world_size(self) -> int:
        raise NotImplementedError

    @property
    def context_and_model_parallel_group(self):
        raise NotImplementedError

    @property
    def cpu_group(self):
        raise NotImplementedError

    def is_data_parallel_head(self) -> bool:
        raise NotImplementedError

    def current_data_parallel_head(self) -> int:
        raise NotImplementedError

    def destroy(self):
        pass

    def train(self, mode: bool = True):
        raise NotImplementedError

    def eval(self):
        return self.train(False)

    def set_version(self, version: int):
        raise NotImplementedError

    def get_version(self) -> int:
        raise NotImplementedError

    def connect_engine(self, engine: "InferenceEngine", meta: WeightUpdateMeta):
        raise NotImplementedError

    def update_weights(self, meta: WeightUpdateMeta):
        raise NotImplementedError

    def get_param_specs(self, weight_chunked_mem_mb: int = 1024) -> list[list[ParamSpec]]:
        raise NotImplementedError

    def save(self, meta: SaveLoadMeta):
        raise NotImplementedError

    def load(self, meta: SaveLoadMeta):
        raise NotImplementedError

    def optimizer_zero_grad(self):
        raise NotImplementedError

    def optimizer_step(self) -> dict[str, float]:
        raise NotImplementedError

    def lr_scheduler_step(self):
        raise NotImplementedError

    def step_lr_scheduler(self):
        return self.lr_scheduler_step()

    def forward_backward_batch(self, mb_list, process_output_fn, forward_only: bool = False):
        raise NotImplementedError

    def train_batch(self, input_: dict[str, Any], loss_fn: Callable, loss_weight_fn: Callable) -> dict[str, float]:
        raise NotImplementedError

    @torch.no_grad()
    def eval_batch(self, input_: dict[str, Any], loss_fn: Callable, loss_weight_fn: Callable):
        raise NotImplementedError

    @torch.no_grad()
    def forward_batch(self, input_: dict[str, Any], output_seqlens=None, aggregate_fn=None):
        raise NotImplementedError

    def forward(self, *args, **kwargs):
        return self.forward_batch(*args, **kwargs)

    def export_stats(self) -> dict[str, float]:
        raise NotImplementedError

    def onload(self):
        raise NotImplementedError

    def offload(self):
        raise NotImplementedError

    def clear_batches(self, *args):
        pass

    def config_perf_tracer(self, config, rank: int, role: str):
        from ..utils import perf_tracer

        perf_tracer.configure(config, rank=rank, role=role)

    def save_perf_tracer(self, step: int | None = None, force: bool = False):
        from ..utils import perf_tracer

        perf_tracer.save(step=step, force=force)

    @property
    def initialized(self) -> bool:
        """True once ``initialize()`` has completed."""
        return bool(getattr(self, "_initialized", False))

    def get_device_stats(self):
        from .io_struct import DeviceRuntimeInfo

        return DeviceRuntimeInfo.get_current()

    def start_memory_profile(self, max_entries: int = 100000) -> None:
        """Starts recording allocator events of this process's device (no-op without CUDA)."""
        import torch

        if torch.cuda.is_available():
            torch.cuda.memory._record_memory_history(max_entries=max_entries)

    def stop_memory_profile(self, snapshot_dir: str) -> None:
        """Dumps the recorded allocator history as ``snapshot_dir/memory_rank{r}.pickle`` and stops recording."""
        import os

        import torch

        if not torch.cuda.is_available():
            return
        os.makedirs(snapshot_dir, exist_ok=True)
        rank = int(os.environ.get("RANK", 0))
        torch.cuda.memory._dump_snapshot(os.path.join(snapshot_dir, f"memory_rank{rank}.pickle"))
        torch.cuda.memory._record_memory_history(enabled=None)

    # rollout through the connected inference engine, with the data management of a model-parallel trainer: the
    # data-parallel heads roll out, the other ranks of a replica receive the head's batch
    def rollout_batch(self, data, workflow=None, workflow_kwargs=None, group_size: int = 1):
        return self._rollout_via_engine("rollout_batch", data, workflow, workflow_kwargs, group_size=group_size)

    def prepare_batch(self, dataloader, workflow=None, workflow_kwargs=None, should_accept_fn=None,
                      group_size: int = 1, dynamic_bs: bool = False):
        return self._rollout_via_engine("prepare_batch", dataloader, workflow, workflow_kwargs,
                                        should_accept_fn=should_accept_fn, group_size=group_size,
                                        dynamic_bs=dynamic_bs)

    def _rollout_via_engine(self, method: str, source, workflow, workflow_kwargs, **kw):
        engine = getattr(self, "rollout_engine", None)
        if engine is None:
            raise RuntimeError(f"{method}() needs a connected inference engine: call connect_engine() first")
        from ..utils.data import broadcast_tensor_container

        batch = None
        if self.is_data_parallel_head():
            batch = getattr(engine, method)(source, workflow, workflow_kwargs, **kw)
        group = self.context_and_model_parallel_group
        if group is None:
            return batch
        return broadcast_tensor_container(batch, src_rank=self.current_data_parallel_head(), group=group)


class InferenceEngine(abc.ABC):
    def initialize(self, *args, **kwargs):
        raise NotImplementedError

    @property
    def initialized(self) -> bool:
        """True once ``initialize()`` has completed (the engine has its workflow executor)."""
        return getattr(self, "_executor", None) is not None

    @property
    def workflow_executor(self):
        """The executor that runs rollout workflows against this engine."""
        ex = getattr(self, "_executor", None)
        if ex is None:
            raise RuntimeError("the engine is not initialized")
        return ex

    def config_perf_tracer(self, config, rank: int, role: str):
        from ..utils import perf_tracer

        perf_tracer.configure(config, rank=rank, role=role)

    def save_perf_tracer(self, step: int | None = None, force: bool = False):
        from ..utils import perf_tracer

        perf_tracer.save(step=step, force=force)

    def destroy(self):
        pass

    async def agenerate(self, req: ModelRequest) -> ModelResponse:
        raise NotImplementedError

    def generate(self, req: ModelRequest) -> ModelResponse:
        import asyncio

        return asyncio.run(self.agenerate(req))

    def init_weights_update_group(self, meta: WeightUpdateMeta) -> Future:
        raise NotImplementedError

    def update_weights_from_distributed(self, meta: WeightUpdateMeta, param_specs: list[ParamSpec]) -> Future:
        raise NotImplementedError

    def update_weights_from_disk(self, meta: WeightUpdateMeta) -> Future:
        raise NotImplementedError

    def set_version(self, version: int):
        raise NotImplementedError

    def get_version(self) -> int:
        raise NotImplementedError

    def submit(self, data: dict[str, Any], workflow=None, workflow_kwargs=None, should_accept_fn=None,
               group_size: int = 1, task_id: int | None = None, callback_addr: str | None = None,
               is_eval: bool = False, proxy_addr: str | None = None) -> int:
        raise NotImplementedError

    def wait(self, count: int, timeout: float | None = None, raise_timeout: bool = True):
        raise NotImplementedError

    def wait_for_task(self, task_id: int, timeout: float | None = None, raise_timeout: bool = True):
        raise NotImplementedError

    def rollout_batch(self, data: list[dict[str, Any]], workflow=None, workflow_kwargs=None,
                      should_accept_fn=None, group_size: int = 1, is_eval: bool = False):
        raise NotImplementedError

    def prepare_batch(self, dataloader, workflow=None, workflow_kwargs=None, should_accept_fn=None,
                      group_size: int = 1, dynamic_bs: bool = False):
        raise NotImplementedError

    def pause(self):
        raise NotImplementedError

    def resume(self):
        raise NotImplementedError

    def pause_generation(self):
        raise NotImplementedError

    def continue_generation(self):
        raise NotImplementedError

    def offload(self):
        raise NotImplementedError

    def onload(self, tags: list[str] | None = None):
        raise NotImplementedError

    def export_stats(self) -> dict[str, float]:
        raise NotImplementedError

    def launch_server(self, server_args: dict[str, Any]):
        raise NotImplementedError

    def teardown_server(self):
        pass
