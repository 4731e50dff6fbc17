"""Per-step profiling hooks shared by the trainers: perf-trace bookkeeping, ``torch.profiler`` captures
at configured steps (merged next to the perf trace) and CUDA memory-history snapshots.

    hooks = StepProfiling(config, rank, role="trainer")
    for step in ...:
        with hooks.step(step):
            ...train...
    hooks.close()

Counterpart of the trainer-side use of PerfTracer / MemoryProfilerConfig in the reference
(areal/utils/perf_tracer.py:1451-1608, areal/engine/megatron_engine.py:1214-1224).
"""

from __future__ import annotations

import contextlib
import os

import torch

from . import logging, perf_tracer

logger = logging.getLogger("StepProfiling")


class StepProfiling:
    def __init__(self, config, rank: int = 0, role: str = "trainer"):
        self.rank = rank
        self.pt_cfg = getattr(config, "perf_tracer", None)
        self.mem_cfg = getattr(config, "memory_profiler", None)
        self.tracer = None
        if self.pt_cfg is not None and self.pt_cfg.enabled:
            self.tracer = perf_tracer.configure(self.pt_cfg, rank, role, device_timing=torch.cuda.is_available())
        self.dir = None
        if self.tracer is not None:
            self.dir = os.path.dirname(self.tracer.path)
        elif self.mem_cfg is not None:
            from ..api.cli_args import get_log_path

            self.dir = get_log_path(config)

    @contextlib.contextmanager
    def step(self, global_step: int):
        if self.tracer is not None:
            self.tracer.set_step(global_step)
        prof = None
        steps = (self.pt_cfg.profile_steps or []) if (self.tracer is not None) else []
        if global_step in steps:
            from torch.profiler import ProfilerActivity, profile

            acts = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if torch.cuda.is_available() else [])
            prof = profile(activities=acts)
            prof.__enter__()
        mem = self.mem_cfg is not None and global_step in (self.mem_cfg.profile_steps or []) and torch.cuda.is_available()
        if mem:
            torch.cuda.memory._record_memory_history(max_entries=self.mem_cfg.max_entries)
        try:
            with perf_tracer.trace_scope(f"train_step_{global_step}", perf_tracer.Category.COMPUTE):
                yield
        finally:
            if prof is not None:
                prof.__exit__(None, None, None)
                out = os.path.join(self.dir, f"torch_profile_step{global_step}_r{self.rank}.json")
                try:
                    prof.export_chrome_trace(out)
                    perf_tracer.instant("torch_profile", perf_tracer.Category.INSTR, {"file": out})
                except Exception as e:  # noqa: BLE001 - profiling must not stop training
                    logger.warning(f"could not export the torch profile: {e}")
            if mem:
                out = os.path.join(self.dir, f"memory_snapshot_step{global_step}_r{self.rank}.pickle")
                try:
                    torch.cuda.memory._dump_snapshot(out)
                finally:
                    torch.cuda.memory._record_memory_history(enabled=None)
            if self.tracer is not None:
                self.tracer.save(global_step)

    def close(self):
        if self.tracer is not None:
            self.tracer.save(force=True)
