"""Frequency-gated evaluation hook (areal/utils/evaluator.py)."""

from __future__ import annotations

from typing import Callable

from ..api.cli_args import EvaluatorConfig
from ..api.io_struct import FinetuneSpec
from .timeutil import EpochStepTimeFreqCtl


class Evaluator:
    def __init__(self, config: EvaluatorConfig, ft_spec: FinetuneSpec | None = None):
        self.config = config
        self.ft_spec = ft_spec
        self.freq_ctl = EpochStepTimeFreqCtl(config.freq_epochs, config.freq_steps, config.freq_secs)

    def state_dict(self):
        return self.freq_ctl.state_dict()

    def load_state_dict(self, s):
        self.freq_ctl.load_state_dict(s)

    def evaluate(self, evaluate_fn: Callable[[], None], epoch: int, step: int, global_step: int) -> bool:
        last_of_epoch = self.ft_spec is not None and step == self.ft_spec.steps_per_epoch - 1
        if not self.freq_ctl.check(epochs=int(last_of_epoch), steps=1):
            return False
        evaluate_fn()
        return True
