"""Helpers for mixing threads and asyncio (areal/infra/utils/concurrent.py in the reference)."""

from __future__ import annotations

import asyncio
import threading
from concurrent.futures import Future
from typing import Any, Awaitable, Callable


def run_async_task(coro_fn: Callable[..., Awaitable[Any]], *args, **kwargs) -> Any:
    """Runs a coroutine to completion from synchronous code, also when a loop is already running
    in this thread (then a helper thread owns a fresh loop)."""
    try:
        asyncio.get_running_loop()
    except RuntimeError:
        return asyncio.run(coro_fn(*args, **kwargs))
    fut: Future = Future()

    def runner():
        try:
            fut.set_result(asyncio.run(coro_fn(*args, **kwargs)))
        except BaseException as e:
            fut.set_exception(e)

    t = threading.Thread(target=runner, daemon=True)
    t.start()
    return fut.result()


async def gather_with_limit(coros, limit: int):
    """``asyncio.gather`` with at most ``limit`` coroutines in flight; keeps the input order."""
    sem = asyncio.Semaphore(limit)

    async def one(c):
        async with sem:
            return await c

    return await asyncio.gather(*[one(c) for c in coros])
