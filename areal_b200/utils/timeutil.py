"""Frequency controllers that decide when to save / evaluate / checkpoint
(areal/utils/timeutil.py:145-182)."""

from __future__ import annotations

import time
from dataclasses import dataclass


@dataclass
class FrequencyControl:
    """Fires every ``frequency_steps`` calls and/or ``frequency_seconds`` seconds."""

    frequency_seconds: float | None = None
    frequency_steps: int | None = None
    initial_value: bool = False

    def __post_init__(self):
        self._last = time.monotonic()
        self._steps = 0
        self._first = self.initial_value

    def check(self, steps: int = 1) -> bool:
        self._steps += steps
        now = time.monotonic()
        if self._first:
            self._first = False
            self._last, self._steps = now, 0
            return True
        fire = False
        if self.frequency_steps is not None and self._steps >= self.frequency_steps:
            fire = True
        if self.frequency_seconds is not None and now - self._last >= self.frequency_seconds:
            fire = True
        if fire:
            self._last, self._steps = now, 0
        return fire

    def state_dict(self):
        return dict(steps=self._steps, elapsed=time.monotonic() - self._last, first=self._first)

    def load_state_dict(self, s):
        self._steps = s["steps"]
        self._last = time.monotonic() - s["elapsed"]
        self._first = s["first"]


class EpochStepTimeFreqCtl:
    """Combines epoch-, step- and time-based triggers; any one fires the action."""

    def __init__(self, freq_epoch: int | None, freq_step: int | None, freq_sec: float | None):
        self.freq_epoch, self.freq_step, self.freq_sec = freq_epoch, freq_step, freq_sec
        self._epoch = FrequencyControl(frequency_steps=freq_epoch)
        self._step = FrequencyControl(frequency_steps=freq_step)
        self._time = FrequencyControl(frequency_seconds=freq_sec)

    def check(self, epochs: int, steps: int) -> bool:
        fired = False
        if self.freq_epoch is not None and epochs > 0 and self._epoch.check(epochs):
            fired = True
        if self.freq_step is not None and self._step.check(steps):
            fired = True
        if self.freq_sec is not None and self._time.check(0):
            fired = True
        if fired:  # an action resets every counter
            for c in (self._epoch, self._step, self._time):
                c._steps, c._last = 0, time.monotonic()
        return fired

    def state_dict(self):
        return dict(epoch=self._epoch.state_dict(), step=self._step.state_dict(), time=self._time.state_dict())

    def load_state_dict(self, s):
        self._epoch.load_state_dict(s["epoch"])
        self._step.load_state_dict(s["step"])
        self._time.load_state_dict(s["time"])


# ------------------------------------------------------------------ value schedules
# Scalars that follow the training step (a KL coefficient, a clip range, a sampling temperature).
import dataclasses as _dc
import math as _math


@_dc.dataclass
class Scheduler:
    """``get(step)`` for ``step`` in ``[0, total_iters]``; steps outside that range are an error."""
    init_value: float
    total_iters: int

    @property
    def final_value(self) -> float:
        return self.get(self.total_iters)

    def get(self, step: int) -> float:
        if step < 0 or step > self.total_iters:
            raise ValueError(f"step {step} outside [0, {self.total_iters}]")
        return float(self._get(step))

    def _get(self, step: int) -> float:
        raise NotImplementedError


@_dc.dataclass
class ConstantScheduler(Scheduler):
    def _get(self, step: int) -> float:
        return self.init_value


@_dc.dataclass
class LinearScheduler(Scheduler):
    end_value: float = 0.0

    def _get(self, step: int) -> float:
        return self.init_value + (self.end_value - self.init_value) * step / max(self.total_iters, 1)


@_dc.dataclass
class ExponentialScheduler(Scheduler):
    decay: float = 1.0

    def _get(self, step: int) -> float:
        return self.init_value * self.decay ** step


@_dc.dataclass
class CosineDecayScheduler(Scheduler):
    end_value: float = 0.0

    def _get(self, step: int) -> float:
        t = step / max(self.total_iters, 1)
        return self.end_value + 0.5 * (self.init_value - self.end_value) * (1 + _math.cos(_math.pi * t))


class ChainedScheduler:
    """Schedules one after the other; each must start where its predecessor ended."""

    def __init__(self, schedulers):
        self.schedulers = list(schedulers)
        for a, b in zip(self.schedulers, self.schedulers[1:]):
            if abs(a.final_value - b.init_value) > 1e-8 * max(1.0, abs(a.final_value)):
                raise ValueError(f"schedule ends at {a.final_value} but the next one starts at {b.init_value}")

    @property
    def total_iters(self) -> int:
        return sum(s.total_iters for s in self.schedulers)

    @property
    def init_value(self) -> float:
        return self.schedulers[0].init_value

    @property
    def final_value(self) -> float:
        return self.schedulers[-1].final_value

    def get(self, step: int) -> float:
        if step < 0 or step > self.total_iters:
            raise ValueError(f"step {step} outside [0, {self.total_iters}]")
        for s in self.schedulers:
            if step <= s.total_iters:
                return s.get(step)
            step -= s.total_iters
        return self.final_value
