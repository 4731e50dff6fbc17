"""Scheduler contract for single-controller mode (areal/api/scheduler_api.py:14-329)."""

from __future__ import annotations

import abc
from dataclasses import dataclass, field
from typing import Any

from .cli_args import SchedulingSpec, SchedulingStrategy


@dataclass
class Worker:
    id: str
    ip: str
    worker_ports: list[str] = field(default_factory=list)
    engine_ports: list[str] = field(default_factory=list)


@dataclass
class Job:
    replicas: int = 0
    tasks: list[SchedulingSpec] = field(default_factory=list)
    scheduling_strategy: SchedulingStrategy = field(default_factory=SchedulingStrategy)
    role: str = "default"


class Scheduler(abc.ABC):
    @abc.abstractmethod
    def create_workers(self, job: Job, *args, **kwargs) -> list[str]:
        """Starts ``job.replicas`` worker processes; returns their ids."""

    @abc.abstractmethod
    def get_workers(self, role: str, timeout: float | None = None) -> list[Worker]:
        """Blocks until every worker of ``role`` answers its health check."""

    @abc.abstractmethod
    def delete_workers(self, role: str | None = None):
        """Stops workers of a role (all roles when ``None``)."""

    def fork_workers(self, role: str, target_role: str, command: str | None = None) -> list[str]:
        raise NotImplementedError

    @abc.abstractmethod
    async def create_engine(self, worker_id: str, engine: str, *args, **kwargs) -> Any:
        """Instantiates ``engine`` (import path) inside the worker."""

    async def set_worker_env(self, worker_id: str, env: dict[str, str]) -> None:
        raise NotImplementedError

    @abc.abstractmethod
    def call_engine(self, worker_id: str, method: str, engine_name: str | None = None, *args, **kwargs) -> Any:
        """Synchronous engine method call with retries."""

    @abc.abstractmethod
    async def async_call_engine(self, worker_id: str, method: str, engine_name: str | None = None,
                                *args, **kwargs) -> Any:
        """Asynchronous engine method call with retries."""
