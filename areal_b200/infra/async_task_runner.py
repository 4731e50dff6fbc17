"""Background asyncio runner: a daemon thread owns an event loop (uvloop when
available); other threads submit coroutine factories and collect results through
thread-safe queues. Supports pause/resume of task *starts*, a bounded input
queue, result waiting with timeout and failure propagation
(behaviour of areal/infra/async_task_runner.py:73-415 in the reference).
"""

from __future__ import annotations

import asyncio
import itertools
import queue
import threading
import time
import traceback
from dataclasses import dataclass, field
from typing import Awaitable, Callable, Generic, TypeVar

from ..utils import logging

logger = logging.getLogger("AsyncTaskRunner")
T = TypeVar("T")


class TaskQueueFullError(RuntimeError):
    pass


@dataclass
class TimedResult(Generic[T]):
    task_id: int
    create_time: float
    data: T
    error: BaseException | None = None
    finish_time: float = field(default_factory=time.monotonic)


class AsyncTaskRunner(Generic[T]):
    def __init__(self, max_queue_size: int = 1 << 16, poll_wait_time: float = 0.02,
                 poll_sleep_time: float = 0.002, enable_tracing: bool = False):
        self.max_queue_size = max_queue_size
        self.poll_wait_time = poll_wait_time
        self.poll_sleep_time = poll_sleep_time
        self._in: queue.Queue = queue.Queue(maxsize=max_queue_size)
        self._out: queue.Queue = queue.Queue()
        self._paused = threading.Event()
        self._exiting = threading.Event()
        self._thread: threading.Thread | None = None
        self._loop: asyncio.AbstractEventLoop | None = None
        self._ready = threading.Event()
        self._error: BaseException | None = None
        self._ids = itertools.count(1)
        self._n_running = 0
        self._lock = threading.Lock()
        self._admit: Callable[[], bool] | None = None

    # ---------------------------------------------------------------- control
    def initialize(self, admit_fn: Callable[[], bool] | None = None):
        """``admit_fn`` (optional) is asked before each task start; returning False delays it."""
        self._admit = admit_fn
        self._thread = threading.Thread(target=self._run, name="async-task-runner", daemon=True)
        self._thread.start()
        if not self._ready.wait(timeout=30):
            raise RuntimeError("task runner thread did not start")

    def destroy(self):
        self._exiting.set()
        if self._thread is not None:
            self._thread.join(timeout=10)
            self._thread = None

    def pause(self):
        self._paused.set()

    def resume(self):
        self._paused.clear()

    def is_paused(self) -> bool:
        return self._paused.is_set()

    def health_check(self):
        if self._error is not None:
            raise RuntimeError("task runner thread died") from self._error
        if self._thread is None or not self._thread.is_alive():
            raise RuntimeError("task runner is not running")

    # ----------------------------------------------------------------- submit
    def submit(self, coro_fn: Callable[..., Awaitable[T]], *args, task_id: int | None = None, **kwargs) -> int:
        self.health_check()
        tid = task_id if task_id is not None else next(self._ids)
        try:
            self._in.put_nowait((tid, time.monotonic(), coro_fn, args, kwargs))
        except queue.Full:
            raise TaskQueueFullError(f"input queue full ({self.max_queue_size}); raise queue_size") from None
        return tid

    def get_input_queue_size(self) -> int:
        return self._in.qsize()

    def get_output_queue_size(self) -> int:
        return self._out.qsize()

    def get_running(self) -> int:
        with self._lock:
            return self._n_running

    # ------------------------------------------------------------------- wait
    def poll(self) -> TimedResult[T] | None:
        try:
            return self._out.get_nowait()
        except queue.Empty:
            return None

    def wait(self, count: int, timeout: float | None = None) -> list[TimedResult[T]]:
        """Blocks until ``count`` results are available (raises ``TimeoutError`` otherwise,
        keeping collected results queued for the next call)."""
        deadline = None if timeout is None else time.monotonic() + timeout
        got: list[TimedResult[T]] = []
        while len(got) < count:
            self.health_check()
            remaining = None if deadline is None else deadline - time.monotonic()
            if remaining is not None and remaining <= 0:
                for r in got:
                    self._out.put(r)
                raise TimeoutError(f"only {len(got)}/{count} results within {timeout}s")
            try:
                got.append(self._out.get(timeout=min(self.poll_wait_time, remaining or self.poll_wait_time)))
            except queue.Empty:
                continue
        return got

    # ------------------------------------------------------------ thread body
    def _run(self):
        try:
            try:
                import uvloop

                loop = uvloop.new_event_loop()
            except Exception:
                loop = asyncio.new_event_loop()
            asyncio.set_event_loop(loop)
            self._loop = loop
            loop.run_until_complete(self._main())
        except BaseException as e:
            self._error = e
            logger.error("task runner crashed:\n" + traceback.format_exc())
        finally:
            self._ready.set()

    async def _main(self):
        self._ready.set()
        tasks: set[asyncio.Task] = set()
        held = None
        while not self._exiting.is_set():
            started = False
            while not self._paused.is_set():
                if held is None:
                    try:
                        held = self._in.get_nowait()
                    except queue.Empty:
                        break
                if self._admit is not None and not self._admit():
                    break
                tid, ctime, fn, args, kwargs = held
                held = None
                t = asyncio.create_task(self._wrap(tid, ctime, fn, args, kwargs))
                tasks.add(t)
                t.add_done_callback(tasks.discard)
                with self._lock:
                    self._n_running += 1
                started = True
            await asyncio.sleep(0 if started else self.poll_sleep_time)
        for t in tasks:
            t.cancel()
        if tasks:
            await asyncio.gather(*tasks, return_exceptions=True)
        # HTTP sessions that workflows opened on this loop end with it
        from .workflow_context import close_clients

        await close_clients()

    async def _wrap(self, tid, ctime, fn, args, kwargs):
        try:
            data = await fn(*args, **kwargs)
            self._out.put(TimedResult(tid, ctime, data))
        except asyncio.CancelledError:
            raise
        except BaseException as e:
            logger.error(f"task {tid} failed: {type(e).__name__}: {e}\n{traceback.format_exc()}")
            self._out.put(TimedResult(tid, ctime, None, error=e))
        finally:
            with self._lock:
                self._n_running -= 1
