"""Per-rank performance tracing in Chrome-trace (Perfetto) JSONL plus a session
tracer for rollout lifecycles.

* ``PerfTracer`` – ``trace_scope`` / ``atrace_scope`` context managers, ``instant``
  events and the ``@trace_perf`` decorator append complete ("X") events to an
  in-memory buffer that ``save`` flushes to ``traces-r{rank}.jsonl`` every
  ``save_interval`` steps. With ``device_timing=True`` a scope is also bracketed
  by CUDA events and the device duration is attached to the event.
* ``SessionTracer`` – records per-rollout sessions (task → session; phases such as
  generate / reward / tool; accepted / rejected) to ``sessions-r{rank}.jsonl``.
* ``convert_jsonl_to_chrome_trace`` merges the per-rank files into one JSON that
  chrome://tracing and Perfetto load.

Counterpart of areal/utils/perf_tracer.py:62-2125 and
areal/tools/perf_trace_converter.py in the reference.
"""

from __future__ import annotations

import contextlib
import functools
import getpass
import glob
import inspect
import json
import os
import threading
import time
from dataclasses import dataclass, field
from enum import Enum
from typing import Any

from ..api.cli_args import PerfTracerConfig, SessionTracerConfig


class Category(str, Enum):
    COMPUTE = "compute"
    COMM = "comm"
    IO = "io"
    SYNC = "sync"
    SCHEDULER = "scheduler"
    INSTR = "instr"
    MISC = "misc"


def _now_us() -> float:
    return time.perf_counter_ns() / 1e3


def _trace_dir(cfg: PerfTracerConfig) -> str:
    d = os.path.join(cfg.fileroot, "logs", getpass.getuser(), cfg.experiment_name, cfg.trial_name, "perf_tracer")
    os.makedirs(d, exist_ok=True)
    return d


class PerfTracer:
    def __init__(self, config: PerfTracerConfig, rank: int = 0, role: str = "trainer", device_timing: bool = False):
        self.config = config
        self.rank, self.role = rank, role
        self.enabled = bool(config.enabled)
        self.device_timing = device_timing
        self._events: list[dict[str, Any]] = []
        self._lock = threading.Lock()
        self._pending_cuda: list[tuple[dict, Any, Any]] = []
        self._step = 0
        self._origin = _now_us()
        self.path = os.path.join(_trace_dir(config), f"traces-r{rank}.jsonl") if self.enabled else None
        self.session_tracer = SessionTracer(config.session_tracer, _trace_dir(config), rank) \
            if (self.enabled and config.session_tracer is not None and config.session_tracer.enabled) else None

    # ------------------------------------------------------------------ events
    def _emit(self, ev: dict[str, Any]):
        ev.setdefault("pid", self.rank)
        ev.setdefault("tid", threading.get_ident() % 100000)
        with self._lock:
            self._events.append(ev)

    def instant(self, name: str, category: Category | str = Category.MISC, args: dict | None = None):
        if self.enabled:
            self._emit(dict(name=name, cat=str(getattr(category, "value", category)), ph="i", s="t",
                            ts=_now_us() - self._origin, args=args or {}))

    @contextlib.contextmanager
    def trace_scope(self, name: str, category: Category | str = Category.MISC, args: dict | None = None):
        if not self.enabled:
            yield
            return
        t0 = _now_us()
        start_ev = end_ev = None
        if self.device_timing:
            import torch

            if torch.cuda.is_available():
                start_ev, end_ev = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                start_ev.record()
        try:
            yield
        finally:
            ev = dict(name=name, cat=str(getattr(category, "value", category)), ph="X", ts=t0 - self._origin,
                      dur=_now_us() - t0, args=dict(args or {}, role=self.role, step=self._step))
            if end_ev is not None:
                end_ev.record()
                with self._lock:
                    self._pending_cuda.append((ev, start_ev, end_ev))
            self._emit(ev)

    @contextlib.asynccontextmanager
    async def atrace_scope(self, name: str, category: Category | str = Category.MISC, args: dict | None = None):
        with self.trace_scope(name, category, args):
            yield

    # -------------------------------------------------------------------- save
    def set_step(self, step: int):
        self._step = step

    def _resolve_device_times(self):
        with self._lock:
            pending, self._pending_cuda = self._pending_cuda, []
        for ev, s, e in pending:
            try:
                e.synchronize()
                ev["args"]["device_ms"] = s.elapsed_time(e)
            except Exception:
                pass

    def save(self, step: int | None = None, force: bool = False):
        if not self.enabled:
            return
        if step is not None:
            self._step = step
        if not force and self.config.save_interval > 0 and (self._step + 1) % self.config.save_interval != 0:
            return
        self._resolve_device_times()
        with self._lock:
            events, self._events = self._events, []
        if events:
            with open(self.path, "a") as f:
                for ev in events:
                    f.write(json.dumps(ev) + "\n")
        if self.session_tracer is not None:
            self.session_tracer.flush(force=True)


_GLOBAL: PerfTracer | None = None


def configure(config: PerfTracerConfig | None, rank: int = 0, role: str = "trainer", device_timing: bool = False):
    global _GLOBAL
    _GLOBAL = PerfTracer(config, rank, role, device_timing) if config is not None else None
    return _GLOBAL


def get_tracer() -> PerfTracer | None:
    return _GLOBAL


def get_session_tracer():
    return _GLOBAL.session_tracer if _GLOBAL is not None else None


@contextlib.contextmanager
def trace_scope(name: str, category: Category | str = Category.MISC, args: dict | None = None):
    if _GLOBAL is None or not _GLOBAL.enabled:
        yield
        return
    with _GLOBAL.trace_scope(name, category, args):
        yield


def instant(name: str, category: Category | str = Category.MISC, args: dict | None = None):
    if _GLOBAL is not None:
        _GLOBAL.instant(name, category, args)


def save(step: int | None = None, force: bool = False):
    if _GLOBAL is not None:
        _GLOBAL.save(step, force)


def trace_perf(name: str | None = None, category: Category | str = Category.MISC):
    """Decorator for sync and async functions."""

    def deco(fn):
        label = name or fn.__qualname__
        if inspect.iscoroutinefunction(fn):
            @functools.wraps(fn)
            async def awrapper(*a, **k):
                with trace_scope(label, category):
                    return await fn(*a, **k)

            return awrapper

        @functools.wraps(fn)
        def wrapper(*a, **k):
            with trace_scope(label, category):
                return fn(*a, **k)

        return wrapper

    return deco


# --------------------------------------------------------------------------- sessions


@dataclass
class SessionRecord:
    session_id: int
    task_id: int | None
    start: float
    end: float | None = None
    status: str = "running"  # running | accepted | rejected | failed
    phases: list[dict[str, Any]] = field(default_factory=list)
    meta: dict[str, Any] = field(default_factory=dict)


class SessionTracer:
    def __init__(self, config: SessionTracerConfig | None, directory: str, rank: int = 0):
        self.config = config or SessionTracerConfig(enabled=True)
        self.path = os.path.join(directory, f"sessions-r{rank}.jsonl")
        self._live: dict[int, SessionRecord] = {}
        self._done: list[SessionRecord] = []
        self._next = 0
        self._lock = threading.Lock()

    def start_session(self, task_id: int | None = None, **meta) -> int:
        with self._lock:
            sid = self._next
            self._next += 1
            self._live[sid] = SessionRecord(sid, task_id, time.time(), meta=dict(meta))
            return sid

    @contextlib.contextmanager
    def phase(self, session_id: int, name: str, **meta):
        t0 = time.time()
        try:
            yield
        finally:
            with self._lock:
                rec = self._live.get(session_id)
                if rec is not None:
                    rec.phases.append(dict(name=name, start=t0, end=time.time(), **meta))

    def end_session(self, session_id: int, status: str = "accepted", **meta):
        with self._lock:
            rec = self._live.pop(session_id, None)
            if rec is None:
                return
            rec.end, rec.status = time.time(), status
            rec.meta.update(meta)
            self._done.append(rec)
            full = len(self._done) >= self.config.flush_threshold
        if full:
            self.flush()

    def flush(self, force: bool = False):
        with self._lock:
            if not self._done:
                return
            done, self._done = self._done, []
        with open(self.path, "a") as f:
            for r in done:
                f.write(json.dumps(dict(session_id=r.session_id, task_id=r.task_id, start=r.start, end=r.end,
                                        status=r.status, phases=r.phases, meta=r.meta)) + "\n")


# --------------------------------------------------------------------------- task / session context
# Workflow code does not carry ids around: the executor binds the task and session of the running episode to the
# coroutine's context, and ``trace_session_phase`` / ``trace_session_event`` anywhere below it (a workflow, an
# agent, a reward call) land in that session's record. Reference: the module-level helpers of
# areal/utils/perf_tracer.py (register_task / register_session, set_/get_task_id, set_/get_session_id,
# session_context, trace_session_phase, atrace_session_phase, trace_session_event).
import contextvars
import itertools

_TASK_ID: contextvars.ContextVar = contextvars.ContextVar("areal_b200_task_id", default=None)
_SESSION_ID: contextvars.ContextVar = contextvars.ContextVar("areal_b200_session_id", default=None)
_task_counter = itertools.count()


def is_configured() -> bool:
    return _GLOBAL is not None and _GLOBAL.enabled


def reset() -> None:
    """Flushes and drops the global tracer (tests; re-configuration inside one process)."""
    global _GLOBAL
    if _GLOBAL is not None:
        _GLOBAL.save(force=True)
    _GLOBAL = None
    _TASK_ID.set(None)
    _SESSION_ID.set(None)


def register_task() -> int:
    """A new task id (one per submitted episode, shared by the sessions that retry it), bound to this context."""
    tid = next(_task_counter)
    _TASK_ID.set(tid)
    return tid


def set_task_id(task_id: int | None) -> None:
    _TASK_ID.set(task_id)


def get_task_id() -> int | None:
    return _TASK_ID.get()


def register_session(task_id: int | None = None, **meta) -> int | None:
    """Starts a session record for ``task_id`` (default: the context's task) and binds it to this context;
    ``None`` when session tracing is off."""
    st = get_session_tracer()
    if st is None:
        return None
    sid = st.start_session(task_id if task_id is not None else _TASK_ID.get(), **meta)
    _SESSION_ID.set(sid)
    return sid


def set_session_id(session_id: int | None) -> None:
    _SESSION_ID.set(session_id)


def get_session_id() -> int | None:
    return _SESSION_ID.get()


@contextlib.contextmanager
def session_context(task_id: int | None = None, **meta):
    """One traced session around a block: registered on entry, ended on exit with status ``accepted`` (``failed``
    if the block raises; set ``ctx["status"]`` inside the block for ``rejected``)."""
    st = get_session_tracer()
    sid = None if st is None else st.start_session(task_id if task_id is not None else _TASK_ID.get(), **meta)
    ctx = {"session_id": sid, "status": "accepted"}
    tok = _SESSION_ID.set(sid)
    try:
        yield ctx
    except BaseException:
        ctx["status"] = "failed"
        raise
    finally:
        _SESSION_ID.reset(tok)
        if st is not None and sid is not None:
            st.end_session(sid, status=ctx["status"])


trace_session = session_context


@contextlib.contextmanager
def trace_session_phase(name: str, **meta):
    """A named phase (generate, reward, tool call ...) of the context's session; a no-op outside a session."""
    st, sid = get_session_tracer(), _SESSION_ID.get()
    if st is None or sid is None:
        yield
        return
    with st.phase(sid, name, **meta):
        yield


@contextlib.asynccontextmanager
async def atrace_session_phase(name: str, **meta):
    with trace_session_phase(name, **meta):
        yield


def trace_session_event(name: str, **meta) -> None:
    """A zero-length phase: marks a moment of the context's session."""
    with trace_session_phase(name, **meta):
        pass


@contextlib.asynccontextmanager
async def atrace_scope(name: str, category: "Category | str" = None, args: dict | None = None):
    with trace_scope(name, category if category is not None else Category.MISC, args):
        yield


PerfTraceCategory = Category


# --------------------------------------------------------------------------- converter


def convert_jsonl_to_chrome_trace(src: str, dst: str | None = None) -> str:
    """``src`` is a directory (all ``traces-r*.jsonl`` inside are merged) or one file."""
    files = sorted(glob.glob(os.path.join(src, "traces-r*.jsonl"))) if os.path.isdir(src) else [src]
    events = []
    for f in files:
        with open(f) as fh:
            events += [json.loads(line) for line in fh if line.strip()]
    events.sort(key=lambda e: e.get("ts", 0))
    dst = dst or (os.path.join(src, "trace.json") if os.path.isdir(src) else os.path.splitext(src)[0] + ".json")
    with open(dst, "w") as f:
        json.dump({"traceEvents": events, "displayTimeUnit": "ms"}, f)
    return dst


if __name__ == "__main__":
    import sys

    print(convert_jsonl_to_chrome_trace(sys.argv[1], sys.argv[2] if len(sys.argv) > 2 else None))
