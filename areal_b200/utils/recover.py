"""Checkpoint-and-resume of a whole training run.

``RecoverHandler.dump`` writes the sharded model + optimizer state
(``recover_checkpoint/``) and a ``RecoverInfo`` record (step position, saver /
evaluator / stats-logger / dataloader state) under ``recover_info/``; ``load``
restores them, re-pushes the weights to the rollout engine and tells the
staleness manager which version it restarts from. The checkpoint is a
``torch.distributed.checkpoint`` directory of named tensors, so a run may resume
at another data-parallel size or parallel layout; generator state is restored
only when the world size is unchanged (areal/utils/recover.py:41-445 in the
reference).
"""

from __future__ import annotations

import getpass
import json
import os
import pickle
from dataclasses import asdict, dataclass, field
from typing import Any

import torch.distributed as dist

from ..api.cli_args import RecoverConfig
from ..api.io_struct import FinetuneSpec, SaveLoadMeta, StepInfo, WeightUpdateMeta
from . import logging
from .timeutil import EpochStepTimeFreqCtl

logger = logging.getLogger("Recover")


class InvalidRecoverInfo(Exception):
    pass


@dataclass
class RecoverInfo:
    last_step_info: StepInfo
    saver_info: dict = field(default_factory=dict)
    evaluator_info: dict = field(default_factory=dict)
    stats_logger_info: dict = field(default_factory=dict)
    dataloader_info: Any = None
    checkpoint_info: dict = field(default_factory=dict)

    def dump(self, root: str):
        os.makedirs(root, exist_ok=True)
        for name in ("saver_info", "evaluator_info", "stats_logger_info", "checkpoint_info"):
            with open(os.path.join(root, f"{name}.json"), "w") as f:
                json.dump(getattr(self, name), f)
        with open(os.path.join(root, "step_info.json"), "w") as f:
            json.dump(asdict(self.last_step_info), f)
        with open(os.path.join(root, "dataloader_info.pkl"), "wb") as f:
            pickle.dump(self.dataloader_info, f)

    @classmethod
    def load(cls, root: str) -> "RecoverInfo":
        try:
            with open(os.path.join(root, "step_info.json")) as f:
                step = StepInfo(**json.load(f))
            vals = {}
            for name in ("saver_info", "evaluator_info", "stats_logger_info", "checkpoint_info"):
                with open(os.path.join(root, f"{name}.json")) as f:
                    vals[name] = json.load(f)
            with open(os.path.join(root, "dataloader_info.pkl"), "rb") as f:
                dl = pickle.load(f)
        except (FileNotFoundError, json.JSONDecodeError, pickle.UnpicklingError, TypeError) as e:
            raise InvalidRecoverInfo(f"recover info under {root} is missing or corrupt: {e}") from e
        return cls(last_step_info=step, dataloader_info=dl, **vals)


class RecoverHandler:
    def __init__(self, config: RecoverConfig, ft_spec: FinetuneSpec | None = None):
        self.config = config
        self.ft_spec = ft_spec
        self.freq_ctl = EpochStepTimeFreqCtl(config.freq_epochs, config.freq_steps, config.freq_secs)

    @staticmethod
    def recover_root(cfg: RecoverConfig) -> str:
        return os.path.join(cfg.fileroot, "checkpoints", getpass.getuser(), cfg.experiment_name, cfg.trial_name)

    def _ckpt_path(self, name="default"):
        return os.path.join(self.recover_root(self.config), name, "recover_checkpoint")

    def _info_path(self):
        return os.path.join(self.recover_root(self.config), "recover_info")

    def dump(self, engine, step_info: StepInfo, saver=None, evaluator=None, stats_logger=None, dataloader=None,
             tokenizer=None, force: bool = False, name: str = "default") -> bool:
        if self.config.mode == "disabled":
            return False
        last_of_epoch = self.ft_spec is not None and step_info.epoch_step == self.ft_spec.steps_per_epoch - 1
        if not force and not self.freq_ctl.check(epochs=int(last_of_epoch), steps=1):
            return False
        path = self._ckpt_path(name)
        engine.save(SaveLoadMeta(path=path, weight_format="dcp", with_optim=not self.config.no_save_optim,
                                 tokenizer=tokenizer))
        if not dist.is_initialized() or dist.get_rank() == getattr(engine, "train_ranks", [0])[0]:
            info = RecoverInfo(
                last_step_info=step_info,
                saver_info=saver.state_dict() if saver is not None else {},
                evaluator_info=evaluator.state_dict() if evaluator is not None else {},
                stats_logger_info=stats_logger.state_dict() if stats_logger is not None else {},
                dataloader_info=dataloader.state_dict() if hasattr(dataloader, "state_dict") else None,
                checkpoint_info={"version": engine.get_version(), "path": path})
            info.dump(self._info_path())
        return True

    def load(self, engine, saver=None, evaluator=None, stats_logger=None, dataloader=None,
             inference_engine=None, weight_update_meta: WeightUpdateMeta | None = None,
             name: str = "default") -> RecoverInfo | None:
        if self.config.mode in ("disabled", "off"):
            return None
        try:
            info = RecoverInfo.load(self._info_path())
        except InvalidRecoverInfo as e:
            if self.config.mode in ("resume", "on"):
                raise
            logger.info(f"no usable recover info ({e}); starting from scratch")
            return None
        engine.load(SaveLoadMeta(path=self._ckpt_path(name), weight_format="dcp",
                                 with_optim=not self.config.no_load_optim))
        version = info.checkpoint_info.get("version", info.last_step_info.global_step + 1)
        engine.set_version(version)
        if saver is not None and info.saver_info:
            saver.load_state_dict(info.saver_info)
        if evaluator is not None and info.evaluator_info:
            evaluator.load_state_dict(info.evaluator_info)
        if stats_logger is not None and info.stats_logger_info:
            stats_logger.load_state_dict(info.stats_logger_info)
        if dataloader is not None and info.dataloader_info is not None and hasattr(dataloader, "load_state_dict"):
            dataloader.load_state_dict(info.dataloader_info)
        if inference_engine is not None and weight_update_meta is not None:
            # the rollout side restarts with the recovered weights and version
            engine.update_weights(weight_update_meta.with_version(version))
            ex = getattr(inference_engine, "_executor", None)
            if ex is not None:
                ex.staleness.on_version_recovered(version)
        logger.info(f"recovered at global step {info.last_step_info.global_step} (version {version})")
        return info


def check_if_auto_recover(config: RecoverConfig) -> bool:
    """Whether a usable recover checkpoint of this experiment / trial exists: the recover info loads, names a step
    that was completed, and the checkpoint directory it points to is there."""
    root = os.path.join(RecoverHandler.recover_root(config), "recover_info")
    try:
        info = RecoverInfo.load(root)
    except InvalidRecoverInfo:
        return False
    if info.last_step_info.global_step < 0:
        return False
    ckpt = (info.checkpoint_info or {}).get("path")
    return ckpt is None or os.path.exists(ckpt)


InValidRecoverInfo = InvalidRecoverInfo  # the spelling used by the reference


def check_if_recover(config: RecoverConfig, run_id: int = 0) -> bool:
    if config.mode in ("disabled", "off"):
        return False
    if config.mode in ("resume", "on"):
        return True
    root = os.path.join(RecoverHandler.recover_root(config), "recover_info")
    exists = os.path.exists(os.path.join(root, "step_info.json"))
    if config.mode == "auto":
        return exists
    if config.mode == "fault":
        return run_id > 0 and exists
    return False
