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
        pass

    def save_perf_tracer(self, step: int | None = None, force: bool = False):
        pass


class InferenceEngine(abc.ABC):
    def initialize(self, *args, **kwargs):
        raise NotImplementedError

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
