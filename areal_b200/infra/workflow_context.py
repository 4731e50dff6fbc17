"""Per-task context of running workflows: which statistics scope a rollout task logs to (train vs
eval), its task id, and HTTP clients that live as long as the event loop that created them.
Counterpart of areal/infra/workflow_context.py in the reference."""

from __future__ import annotations

import asyncio
import contextvars
from contextlib import contextmanager
from dataclasses import dataclass
from typing import Any


@dataclass
class WorkflowContext:
    is_eval: bool = False
    task_id: int | None = None
    stat_scope_name: str | None = None


_ctx: contextvars.ContextVar[WorkflowContext] = contextvars.ContextVar("areal_b200_workflow_ctx", default=WorkflowContext())
_clients: dict[tuple[int, str], Any] = {}


def get() -> WorkflowContext:
    return _ctx.get()


def set(ctx: WorkflowContext):  # noqa: A001 - mirrors the reference's module-level API
    return _ctx.set(ctx)


@contextmanager
def scope(is_eval: bool = False, task_id: int | None = None, stat_scope_name: str | None = None):
    tok = _ctx.set(WorkflowContext(is_eval, task_id, stat_scope_name))
    try:
        yield
    finally:
        _ctx.reset(tok)


def stat_scope() -> str:
    c = _ctx.get()
    return c.stat_scope_name or ("eval-rollout" if c.is_eval else "rollout")


async def get_aiohttp_session():
    """One ``aiohttp.ClientSession`` per event loop (sessions must not cross loops)."""
    import aiohttp

    loop = asyncio.get_running_loop()
    key = (id(loop), "aiohttp")
    s = _clients.get(key)
    if s is None or s.closed:
        s = aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=3600), connector=aiohttp.TCPConnector(limit=0))
        _clients[key] = s
    return s


async def close_clients():
    loop = asyncio.get_running_loop()
    for key in [k for k in _clients if k[0] == id(loop)]:
        s = _clients.pop(key)
        try:
            await s.close()
        except Exception:
            pass
