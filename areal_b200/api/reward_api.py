"""Asynchronous wrapper around synchronous reward functions.

Reward functions can be slow or crash-prone (symbolic math checkers, code
execution), so they run in a process pool with a timeout, bounded retries and a
rebuild of the pool when a worker dies (behaviour of areal/api/reward_api.py:63-209).
"""

from __future__ import annotations

import asyncio
import concurrent.futures as cf
import multiprocessing
import threading
from concurrent.futures.process import BrokenProcessPool
from typing import Any, Callable

from ..utils import logging

logger = logging.getLogger("Reward")


class AsyncRewardWrapper:
    _pools: dict[int, cf.ProcessPoolExecutor] = {}
    _refs: dict[int, int] = {}
    _lock = threading.Lock()

    def __init__(self, reward_fn: Callable[..., float], timeout_seconds: float = 15.0,
                 max_workers: int | None = None, max_retries: int = 3, default: float = 0.0):
        self.reward_fn = reward_fn
        self.timeout = timeout_seconds
        self.max_workers = max_workers or 4
        self.max_retries = max_retries
        self.default = default
        with self._lock:
            if self.max_workers not in self._pools:
                self._pools[self.max_workers] = _new_pool(self.max_workers)
                self._refs[self.max_workers] = 0
            self._refs[self.max_workers] += 1

    def _pool(self) -> cf.ProcessPoolExecutor:
        with self._lock:
            if self.max_workers not in self._pools:
                self._pools[self.max_workers] = _new_pool(self.max_workers)
            return self._pools[self.max_workers]

    def _rebuild(self):
        with self._lock:
            old = self._pools.pop(self.max_workers, None)
            if old is not None:
                old.shutdown(wait=False, cancel_futures=True)
            self._pools[self.max_workers] = _new_pool(self.max_workers)

    async def __call__(self, *args: Any, **kwargs: Any) -> float:
        loop = asyncio.get_running_loop()
        for attempt in range(self.max_retries + 1):
            try:
                fut = loop.run_in_executor(self._pool(), _call, self.reward_fn, args, kwargs)
                return float(await asyncio.wait_for(fut, timeout=self.timeout))
            except asyncio.TimeoutError:
                logger.warning(f"reward function timed out after {self.timeout}s; returning {self.default}")
                return self.default
            except BrokenProcessPool:
                logger.warning(f"reward pool broke (attempt {attempt + 1}); rebuilding")
                self._rebuild()
            except Exception as e:  # the reward function raised: treat as a failed sample
                logger.warning(f"reward function raised {type(e).__name__}: {e}")
                return self.default
        return self.default

    def __del__(self):
        try:
            with self._lock:
                n = self._refs.get(self.max_workers, 0) - 1
                self._refs[self.max_workers] = n
                if n <= 0:
                    pool = self._pools.pop(self.max_workers, None)
                    if pool is not None:
                        pool.shutdown(wait=False, cancel_futures=True)
        except Exception:
            pass


def _new_pool(n: int) -> cf.ProcessPoolExecutor:
    # "spawn": the callers are multi-threaded processes that hold a CUDA context; forking one of those
    # hands the child locks and device state it must not touch
    return cf.ProcessPoolExecutor(n, mp_context=multiprocessing.get_context("spawn"))


def _call(fn, args, kwargs):
    return fn(*args, **kwargs)
