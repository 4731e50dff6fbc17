"""Periodic HF-format export of the trained weights
(areal/utils/saver.py:35-120; layout ``{fileroot}/checkpoints/{user}/{exp}/{trial}/{name}/epoch{E}epochstep{S}globalstep{G}``)."""

from __future__ import annotations

import getpass
import os

from ..api.cli_args import SaverConfig
from ..api.io_struct import FinetuneSpec, SaveLoadMeta
from .timeutil import EpochStepTimeFreqCtl


class Saver:
    def __init__(self, config: SaverConfig, ft_spec: FinetuneSpec | None = None):
        self.config = config
        self.ft_spec = ft_spec
        self.freq_ctl = EpochStepTimeFreqCtl(config.freq_epochs, config.freq_steps, config.freq_secs)

    @staticmethod
    def get_save_root(experiment_name: str, trial_name: str, fileroot: str) -> str:
        return os.path.join(fileroot, "checkpoints", getpass.getuser(), experiment_name, trial_name)

    @staticmethod
    def get_model_save_root(experiment_name: str, trial_name: str, fileroot: str, name: str = "default") -> str:
        return os.path.join(Saver.get_save_root(experiment_name, trial_name, fileroot), name)

    @staticmethod
    def get_model_save_path(experiment_name, trial_name, fileroot, epoch, step, globalstep, name="default") -> str:
        return os.path.join(Saver.get_model_save_root(experiment_name, trial_name, fileroot, name),
                            f"epoch{epoch}epochstep{step}globalstep{globalstep}")

    def state_dict(self):
        return self.freq_ctl.state_dict()

    def load_state_dict(self, s):
        self.freq_ctl.load_state_dict(s)

    def save(self, engine, epoch: int, step: int, global_step: int, name: str = "default", tokenizer=None,
             processor=None, base_model_path=None, force: bool = False) -> str | None:
        last_of_epoch = self.ft_spec is not None and step == self.ft_spec.steps_per_epoch - 1
        if not force and not self.freq_ctl.check(epochs=int(last_of_epoch), steps=1):
            return None
        c = self.config
        path = self.get_model_save_path(c.experiment_name, c.trial_name, c.fileroot, epoch, step, global_step, name)
        engine.save(SaveLoadMeta(path=path, weight_format="hf", with_optim=False, tokenizer=tokenizer,
                                 processor=processor, base_model_path=base_model_path))
        return path
