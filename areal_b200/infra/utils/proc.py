"""Process helpers: terminate exactly the process tree that this process started (by pid, never
by name pattern). Reference: areal/infra/utils/proc.py."""

from __future__ import annotations

import os
import signal
import subprocess
import time

import psutil


def kill_process_tree(pid: int, timeout: float = 10.0, include_parent: bool = True) -> int:
    """SIGTERM, then SIGKILL after ``timeout``, for ``pid`` and all its descendants. Returns the
    number of processes signalled."""
    try:
        parent = psutil.Process(pid)
    except psutil.NoSuchProcess:
        return 0
    procs = parent.children(recursive=True) + ([parent] if include_parent else [])
    for p in procs:
        try:
            p.send_signal(signal.SIGTERM)
        except psutil.NoSuchProcess:
            pass
    _, alive = psutil.wait_procs(procs, timeout=timeout)
    for p in alive:
        try:
            p.kill()
        except psutil.NoSuchProcess:
            pass
    return len(procs)


def run_with_streaming_logs(cmd: list[str], log_path: str, env: dict | None = None) -> subprocess.Popen:
    os.makedirs(os.path.dirname(log_path) or ".", exist_ok=True)
    f = open(log_path, "a")
    return subprocess.Popen(cmd, stdout=f, stderr=subprocess.STDOUT, env=env, start_new_session=True)


def wait_for(predicate, timeout: float, interval: float = 0.1, what: str = "condition"):
    deadline = time.monotonic() + timeout
    while not predicate():
        if time.monotonic() > deadline:
            raise TimeoutError(f"timed out after {timeout}s waiting for {what}")
        time.sleep(interval)
