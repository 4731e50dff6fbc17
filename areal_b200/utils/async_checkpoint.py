"""Asynchronous checkpoint writes: the state is staged to (pinned) host memory on the caller's
thread, the file write runs on a background thread, and at most one write is in flight (the next
save waits for the previous one). Reference: areal/utils/async_checkpoint.py."""

from __future__ import annotations

import os
import threading
from concurrent.futures import Future, ThreadPoolExecutor
from typing import Any, Callable

import torch


def _to_host(obj: Any) -> Any:
    if torch.is_tensor(obj):
        if obj.is_cuda:
            host = torch.empty(obj.shape, dtype=obj.dtype, pin_memory=True)
            host.copy_(obj, non_blocking=True)
            return host
        return obj.detach().clone()
    if isinstance(obj, dict):
        return {k: _to_host(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return type(obj)(_to_host(v) for v in obj)
    return obj


class AsyncCheckpointer:
    def __init__(self):
        self._pool = ThreadPoolExecutor(max_workers=1, thread_name_prefix="ckpt")
        self._pending: Future | None = None
        self._lock = threading.Lock()

    def save(self, state: Any, path: str, writer: Callable[[Any, str], None] | None = None) -> Future:
        """Stages ``state`` and schedules the write; returns the future of the write."""
        self.wait()
        staged = _to_host(state)
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        writer = writer or self._torch_save
        with self._lock:
            self._pending = self._pool.submit(writer, staged, path)
        return self._pending

    @staticmethod
    def _torch_save(state, path):
        os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
        tmp = path + ".tmp"
        torch.save(state, tmp)
        os.replace(tmp, path)  # readers never see a partial file

    def wait(self):
        with self._lock:
            f, self._pending = self._pending, None
        if f is not None:
            f.result()

    def close(self):
        self.wait()
        self._pool.shutdown(wait=True)
