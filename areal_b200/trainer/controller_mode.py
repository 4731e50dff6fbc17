"""Single-controller mode of the PPO / GRPO trainer.

With ``scheduler.type: local`` (or ``slurm`` / ``ray``) the script that creates ``PPOTrainer`` is ONE
controller process that owns no model. It asks the scheduler for workers, creates a train engine in each
trainer worker (``TrainController`` over ``PPOActorEngine``) and a rollout engine in each rollout worker
(``RolloutController`` over ``NativeRolloutEngine``), and then runs the same loop as the SPMD trainer with
every engine call turned into a fan-out RPC: batches travel as ``RTensor`` handles, statistics come back
merged. Weight updates go through a checkpoint directory: the trainer workers write HF safetensors, the
rollout workers load them, the controller orders pause → save → load → version bump → resume.

Reference: areal/trainer/rl_trainer.py:121-123,876,933-1041 (``_init_scheduler``, ``Engine.as_controller``),
areal/infra/controller/train_controller.py:336-384, areal/infra/controller/rollout_controller.py:158-311.
"""

from __future__ import annotations

import os
import time
from typing import Any

import torch

from ..api.alloc_mode import ModelAllocation
from ..api.cli_args import PPOConfig
from ..api.io_struct import FinetuneSpec, SaveLoadMeta, WeightUpdateMeta
from ..infra.controller.rollout_controller import RolloutController
from ..infra.controller.train_controller import TrainController
from ..utils import logging, stats_tracker
from ..utils.stats_logger import StatsLogger

logger = logging.getLogger("PPOTrainer")

ACTOR_ENGINE = "areal_b200.trainer.ppo.actor.PPOActorEngine"
ROLLOUT_ENGINE = "areal_b200.engine.rollout_engine.NativeRolloutEngine"


def make_scheduler(config: PPOConfig):
    kind = config.scheduler.type
    log_dir = os.path.join(config.cluster.fileroot, "logs", str(config.experiment_name), str(config.trial_name))
    if kind == "local":
        from ..infra.scheduler.local import LocalScheduler

        gpus = list(range(torch.cuda.device_count())) if torch.cuda.is_available() else []
        return LocalScheduler(gpu_devices=gpus, log_dir=log_dir)
    if kind == "slurm":
        from ..infra.scheduler.slurm import SlurmScheduler

        return SlurmScheduler(config)
    if kind == "ray":
        from ..infra.scheduler.ray import RayScheduler

        return RayScheduler(config)
    raise ValueError(f"unknown scheduler type {kind!r}")


class ControllerPPOTrainer:
    def __init__(self, config: PPOConfig, train_dataset, valid_dataset=None, tokenizer=None, processor=None,
                 scheduler=None):
        from .rl_trainer import _ListLoader

        self.config, self.tokenizer = config, tokenizer
        self.train_dataset, self.valid_dataset = train_dataset, valid_dataset
        self.scheduler = scheduler or make_scheduler(config)
        self.actor_alloc = ModelAllocation.from_str(config.actor.backend)
        self.rollout_alloc = ModelAllocation.from_str(config.rollout.backend)
        bs = config.train_dataset.batch_size
        self.ft_spec = FinetuneSpec(total_train_epochs=config.total_train_epochs, dataset_size=len(train_dataset),
                                    train_batch_size=bs)
        group = config.gconfig.n_samples
        config.rollout.consumer_batch_size = bs
        self.rollout = RolloutController(ROLLOUT_ENGINE, config.rollout, self.scheduler)
        self.rollout.initialize(role="rollout", alloc_mode=self.rollout_alloc)
        self.actor = TrainController(ACTOR_ENGINE, config.actor, self.scheduler)
        self.actor.initialize(role="actor", alloc_mode=self.actor_alloc, ft_spec=self.ft_spec, group_size=group,
                              seed=config.seed)
        self.weight_root = os.path.join(config.cluster.fileroot, "weight_update", str(config.experiment_name),
                                        str(config.trial_name))
        self.dataloader = _ListLoader(train_dataset, bs, config.train_dataset.shuffle, config.seed)
        self.stats_logger = StatsLogger(config, self.ft_spec)
        self.trained_tokens = 0
        self.last_batch: dict[str, Any] | None = None
        self.is_trainer = True
        self.rank = 0

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def close(self):
        for c in (getattr(self, "actor", None), getattr(self, "rollout", None)):
            if c is not None:
                c.destroy()
        if getattr(self, "stats_logger", None) is not None:
            self.stats_logger.close()

    def _sync_weights(self, version: int) -> float:
        """pause → trainer workers write a checkpoint → rollout workers load it → new version → resume."""
        t0 = time.perf_counter()
        vdir = os.path.join(self.weight_root, f"weight_update_v{version}")
        self.rollout.pause_generation()
        self.actor.save(SaveLoadMeta(path=vdir, weight_format="hf", with_optim=False))
        self.rollout.update_weights_from_disk(WeightUpdateMeta(type="disk", path=vdir, version=version)).result()
        self.rollout.set_version(version)
        self.actor.set_version(version)
        self.rollout.continue_generation()
        prev = getattr(self, "_last_weight_dir", None)
        if prev and prev != vdir and os.path.isdir(prev):
            import shutil

            shutil.rmtree(prev, ignore_errors=True)
        self._last_weight_dir = vdir
        return time.perf_counter() - t0

    def train(self, workflow, workflow_kwargs: dict | None = None, eval_workflow=None, eval_workflow_kwargs=None,
              max_steps: int | None = None, step_callback=None):
        cfg = self.config
        total = cfg.total_train_steps or self.ft_spec.total_train_steps
        if max_steps is not None:
            total = min(total, max_steps)
        group = cfg.gconfig.n_samples
        self._sync_weights(0)  # both sides start from the trainer's weights
        steps_per_epoch = self.ft_spec.steps_per_epoch
        for global_step in range(total):
            epoch, epoch_step = divmod(global_step, steps_per_epoch)
            with stats_tracker.record_timing("rollout"):
                batch = self.rollout.prepare_batch(self.dataloader, workflow, workflow_kwargs, group_size=group)
            self.last_batch = batch
            if cfg.actor.should_compute_prox_logp():
                with stats_tracker.record_timing("recompute_logp"):
                    batch["prox_logp"] = self.actor.compute_logp(batch)
            with stats_tracker.record_timing("compute_advantage"):
                adv_batch = self.actor.compute_advantages(batch)
            with stats_tracker.record_timing("train_step"):
                train_stats = self.actor.ppo_update(adv_batch)
            self.actor.clear_batches()
            n_tok = int(batch["attention_mask"].sum())
            self.trained_tokens += n_tok
            with stats_tracker.record_timing("update_weights"):
                sync_s = self._sync_weights(global_step + 1)
            last = train_stats[-1] if isinstance(train_stats, list) else train_stats
            out = {"step/trained_tokens": float(n_tok), "step/weight_sync_s": float(sync_s),
                   "step/loss": float(last.get("loss", 0.0)), "step/grad_norm": float(last.get("grad_norm", 0.0))}
            exported = stats_tracker.export_all()
            exported.update(out)
            self.stats_logger.commit(epoch, epoch_step, global_step, exported)
            if step_callback is not None:
                step_callback(global_step, exported)
