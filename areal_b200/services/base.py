"""Shared pieces of the micro-services: bearer-token authentication, the worker registry with
placement strategies (round robin, least loaded, session affinity) and a forwarding helper.
Reference: areal/experimental/inference_service/router/{app,strategies}.py,
areal/experimental/agent_service/auth.py."""

from __future__ import annotations

import hmac
import itertools
import threading
import time
from dataclasses import dataclass, field
from typing import Any, Callable

from fastapi import HTTPException, Request


def make_auth(token: str | None) -> Callable[[Request], None]:
    """FastAPI dependency body: rejects requests whose ``Authorization: Bearer`` token differs
    (constant-time compare). ``token=None`` turns authentication off."""

    def check(req: Request):
        if token is None:
            return
        got = req.headers.get("authorization", "")
        if not got.lower().startswith("bearer ") or not hmac.compare_digest(got[7:].strip(), token):
            raise HTTPException(status_code=401, detail="invalid or missing bearer token")

    return check


@dataclass
class WorkerEntry:
    worker_id: str
    addr: str
    inflight: int = 0
    healthy: bool = True
    last_seen: float = field(default_factory=time.time)
    meta: dict = field(default_factory=dict)


class WorkerRegistry:
    """Thread-safe registry + placement. ``pick(session_id)`` keeps a session on its worker."""

    def __init__(self, strategy: str = "round_robin", heartbeat_timeout: float | None = None):
        if strategy not in ("round_robin", "least_loaded"):
            raise ValueError(f"unknown routing strategy {strategy!r}")
        self.strategy, self.heartbeat_timeout = strategy, heartbeat_timeout
        self._workers: dict[str, WorkerEntry] = {}
        self._sessions: dict[str, str] = {}
        self._rr = itertools.count()
        self._lock = threading.Lock()

    def register(self, worker_id: str, addr: str, **meta) -> WorkerEntry:
        with self._lock:
            e = self._workers.get(worker_id)
            if e is None:
                e = self._workers[worker_id] = WorkerEntry(worker_id, addr, meta=meta)
            e.addr, e.healthy, e.last_seen = addr, True, time.time()
            e.meta.update(meta)
            return e

    def unregister(self, worker_id: str):
        with self._lock:
            self._workers.pop(worker_id, None)
            for s in [s for s, w in self._sessions.items() if w == worker_id]:
                del self._sessions[s]

    def heartbeat(self, worker_id: str) -> bool:
        with self._lock:
            e = self._workers.get(worker_id)
            if e is None:
                return False
            e.last_seen, e.healthy = time.time(), True
            return True

    def mark_unhealthy(self, worker_id: str):
        with self._lock:
            if worker_id in self._workers:
                self._workers[worker_id].healthy = False

    def _alive(self) -> list[WorkerEntry]:
        now = time.time()
        return [w for w in self._workers.values() if w.healthy and
                (self.heartbeat_timeout is None or now - w.last_seen <= self.heartbeat_timeout)]

    def pick(self, session_id: str | None = None) -> WorkerEntry:
        with self._lock:
            alive = self._alive()
            if not alive:
                raise HTTPException(status_code=503, detail="no healthy worker is registered")
            if session_id is not None:
                wid = self._sessions.get(session_id)
                e = self._workers.get(wid) if wid else None
                if e is not None and e in alive:
                    return e
            if self.strategy == "least_loaded":
                e = min(alive, key=lambda w: (w.inflight, w.worker_id))
            else:
                alive.sort(key=lambda w: w.worker_id)
                e = alive[next(self._rr) % len(alive)]
            if session_id is not None:
                self._sessions[session_id] = e.worker_id
            return e

    def end_session(self, session_id: str):
        with self._lock:
            self._sessions.pop(session_id, None)

    def acquire(self, e: WorkerEntry):
        with self._lock:
            e.inflight += 1

    def release(self, e: WorkerEntry):
        with self._lock:
            e.inflight = max(0, e.inflight - 1)

    def snapshot(self) -> list[dict[str, Any]]:
        with self._lock:
            return [dict(worker_id=w.worker_id, addr=w.addr, inflight=w.inflight, healthy=w.healthy, **w.meta)
                    for w in sorted(self._workers.values(), key=lambda w: w.worker_id)]


def forward(registry: WorkerRegistry, path: str, payload: Any, session_id: str | None = None,
            post: Callable[[str, Any], Any] | None = None, retries: int = 1) -> Any:
    """Sends ``payload`` to a picked worker; on a transport error the worker is marked unhealthy
    and another one is tried (sessions lose their affinity in that case)."""
    from ..infra.utils.http import HTTPRequestError, request_with_retry

    post = post or (lambda url, body: request_with_retry("POST", url, json=body, max_retries=0).json())
    last: Exception | None = None
    for _ in range(retries + 1):
        e = registry.pick(session_id)
        registry.acquire(e)
        try:
            return post(f"http://{e.addr}{path}" if not e.addr.startswith("http") else e.addr + path, payload)
        except HTTPRequestError as err:
            last = err
            if err.status is not None and err.status < 500:
                raise
            registry.mark_unhealthy(e.worker_id)
        finally:
            registry.release(e)
    raise HTTPException(status_code=502, detail=f"all workers failed: {last}")
