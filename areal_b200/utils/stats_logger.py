"""Rank-0 sink for exported statistics: console table, JSONL file, and TensorBoard /
Weights & Biases / SwanLab / Trackio when those packages are importable and enabled
(areal/utils/stats_logger.py). A backend that fails to start is logged and left out; it
never stops the run."""

from __future__ import annotations

import getpass
import json
import os
import time

import torch.distributed as dist

from ..api.cli_args import StatsLoggerConfig
from ..api.io_struct import FinetuneSpec
from . import logging

logger = logging.getLogger("StatsLogger")


class StatsLogger:
    def __init__(self, config, ft_spec: FinetuneSpec | None = None):
        # accepts either the full experiment config or a StatsLoggerConfig
        self.exp_config = config if hasattr(config, "stats_logger") else None
        self.config: StatsLoggerConfig = config.stats_logger if hasattr(config, "stats_logger") else config
        self.ft_spec = ft_spec
        self._last = time.perf_counter()
        self._tb = None
        self._wandb = None
        self._swanlab = None
        self._trackio = None
        self._file = None
        self._start = time.perf_counter()
        if self._is_main():
            self._init()

    @staticmethod
    def _is_main() -> bool:
        return not dist.is_initialized() or dist.get_rank() == 0

    @staticmethod
    def get_log_path(config: StatsLoggerConfig) -> str:
        path = os.path.join(config.fileroot, "logs", getpass.getuser(), config.experiment_name,
                            config.trial_name)
        os.makedirs(path, exist_ok=True)
        return path

    def _init(self):
        path = self.get_log_path(self.config)
        self._file = open(os.path.join(path, "stats.jsonl"), "a")
        tb_path = self.config.tensorboard.path
        if tb_path:
            try:
                from torch.utils.tensorboard import SummaryWriter

                self._tb = SummaryWriter(log_dir=tb_path)
            except Exception as e:  # tensorboard is optional
                logger.warning(f"tensorboard disabled: {e}")
        if self.config.wandb.mode != "disabled":
            try:
                import wandb

                wandb.init(mode=self.config.wandb.mode, project=self.config.wandb.project or
                           self.config.experiment_name, name=self.config.wandb.name or self.config.trial_name,
                           config=self.config.wandb.config, dir=path)
                self._wandb = wandb
            except Exception as e:
                logger.warning(f"wandb disabled: {e}")
        sw = self.config.swanlab
        if (sw.mode or "disabled") != "disabled":
            try:
                import swanlab

                if sw.api_key:
                    swanlab.login(sw.api_key)
                swanlab.init(project=sw.project or self.config.experiment_name, experiment_name=sw.name or
                             self.config.trial_name, config=sw.config, logdir=sw.logdir or path, mode=sw.mode)
                self._swanlab = swanlab
            except Exception as e:
                logger.warning(f"swanlab disabled: {e}")
        tk = self.config.trackio
        if (tk.mode or "disabled") != "disabled":
            try:
                import trackio

                kw = {"space_id": tk.space_id} if tk.space_id else {}
                trackio.init(project=tk.project or self.config.experiment_name, name=tk.name or
                             self.config.trial_name, **kw)
                self._trackio = trackio
            except Exception as e:
                logger.warning(f"trackio disabled: {e}")

    def state_dict(self):
        return {"last_commit": self._last}

    def load_state_dict(self, s):
        self._last = s.get("last_commit", self._last)

    def commit(self, epoch: int, step: int, global_step: int, data: dict | list[dict]):
        if not self._is_main():
            return
        items = data if isinstance(data, list) else [data]
        now = time.perf_counter()
        logger.info(f"Epoch {epoch + 1} step {step + 1} (global step {global_step + 1}) finished in "
                    f"{now - self._last:.2f}s; {now - self._start:.1f}s since start.")
        self._last = now
        for i, item in enumerate(items):
            gs = global_step * len(items) + i
            logger.info("\n" + self._table(item))
            if self._file:
                self._file.write(json.dumps({"global_step": gs, **{k: float(v) for k, v in item.items()}}) + "\n")
                self._file.flush()
            if self._tb:
                for k, v in item.items():
                    self._tb.add_scalar(k, v, gs)
            if self._wandb:
                self._wandb.log(item, step=gs)
            if self._swanlab:
                self._swanlab.log(item, step=gs)
            if self._trackio:
                self._trackio.log(item, step=gs)

    @staticmethod
    def _table(d: dict) -> str:
        if not d:
            return "(no stats)"
        w = max(len(k) for k in d)
        return "\n".join(f"  {k.ljust(w)}  {v:.6g}" for k, v in sorted(d.items()))

    def close(self):
        if self._file:
            self._file.close()
        if self._tb:
            self._tb.close()
        if self._wandb:
            self._wandb.finish()
        if self._swanlab:
            self._swanlab.finish()
        if self._trackio:
            self._trackio.finish()
