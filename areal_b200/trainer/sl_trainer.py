"""Supervised trainers: SFT, reward model, DPO.

All three share one loop — dataloader → collate to a padded batch → engine step →
save / evaluate / recover / log — and differ in the engine wrapper and the
collate function (areal/trainer/{sft,rw,dpo}_trainer.py in the reference).
"""

from __future__ import annotations

import os
import time
from typing import Any, Callable

import torch
import torch.distributed as dist

from ..api.alloc_mode import ModelAllocation
from ..api.cli_args import RWConfig
from ..api.io_struct import FinetuneSpec, StepInfo
from ..engine.train_engine import B200TrainEngine
from ..utils import logging, seeding, stats_tracker
from ..utils.data import pad_sequences_to_tensors
from ..utils.evaluator import Evaluator
from ..utils.recover import RecoverHandler
from ..utils.saver import Saver
from ..utils.stats_logger import StatsLogger
from .dpo.dpo_engine import DPOEngine
from .rl_trainer import _ListLoader
from .rw.rw_engine import RWEngine
from .sft.lm_engine import LMEngine

logger = logging.getLogger("SLTrainer")


def collate_sft(items: list[dict[str, Any]]) -> dict[str, torch.Tensor]:
    """Items carry ``input_ids`` and ``loss_mask`` (1 on answer tokens); vision-language items also
    ``multi_modal_input`` (a one-element list with the image processor's ``pixel_values`` / ``image_grid_thw``),
    which becomes one dict per row of the batch."""
    batch = pad_sequences_to_tensors([dict(input_ids=torch.as_tensor(x["input_ids"]),
                                           loss_mask=torch.as_tensor(x["loss_mask"])) for x in items])
    if any(x.get("multi_modal_input") for x in items):
        mm = []
        for x in items:
            v = x.get("multi_modal_input") or {}
            mm.append(v[0] if isinstance(v, (list, tuple)) else v)
        batch["multi_modal_input"] = mm
    return batch


def collate_pairs(items: list[dict[str, Any]]) -> dict[str, torch.Tensor]:
    """Items carry ``chosen_ids`` / ``rejected_ids`` (and optional masks); rows are interleaved."""
    rows = []
    for x in items:
        for key in ("chosen", "rejected"):
            ids = torch.as_tensor(x[f"{key}_ids"])
            mask = torch.as_tensor(x.get(f"{key}_loss_mask", [1] * len(ids)))
            rows.append(dict(input_ids=ids, loss_mask=mask))
    return pad_sequences_to_tensors(rows)


class _SLTrainer:
    collate: Callable = staticmethod(collate_sft)

    def __init__(self, config, train_dataset, valid_dataset=None, tokenizer=None, processor=None):
        self.tokenizer = tokenizer
        self.processor = processor  # vision-language models: saved next to the weights
        self.config = config
        use_cuda = torch.cuda.is_available()
        if not dist.is_initialized() and "RANK" in os.environ:
            import datetime

            if use_cuda:
                torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
            dist.init_process_group(backend="nccl" if use_cuda else "gloo",
                                    timeout=datetime.timedelta(seconds=7200))
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        seeding.set_random_seed(config.seed, f"trainer{self.rank}")
        actor_cfg = config.actor if getattr(config, "model", None) is None else config.model
        self.alloc = ModelAllocation.from_str(actor_cfg.backend)
        bs = config.train_dataset.batch_size
        self.ft_spec = FinetuneSpec(config.total_train_epochs, len(train_dataset), bs)
        self.engine = B200TrainEngine(actor_cfg)
        self.engine.create_process_group(self.alloc.parallel)
        self.engine.initialize(None, self.ft_spec, seed=config.seed)
        self.train_loader = _ListLoader(train_dataset, max(bs // self.world, 1), config.train_dataset.shuffle,
                                        config.seed, self.rank, self.world)
        self.valid_loader = None
        if valid_dataset is not None:
            vbs = config.valid_dataset.batch_size if config.valid_dataset else bs
            self.valid_loader = _ListLoader(valid_dataset, max(vbs // self.world, 1), False, config.seed, self.rank,
                                            self.world, drop_last=False)
        self.saver = Saver(config.saver, self.ft_spec)
        self.evaluator = Evaluator(config.evaluator, self.ft_spec)
        self.recover = RecoverHandler(config.recover, self.ft_spec)
        self.stats_logger = StatsLogger(config, self.ft_spec) if self.rank == 0 else None
        self.wrapper = self._make_wrapper(actor_cfg)
        from ..utils.step_profiling import StepProfiling

        self.profiling = StepProfiling(config, self.rank, "trainer")

    def _make_wrapper(self, actor_cfg):
        raise NotImplementedError

    def _train_step(self, batch) -> dict[str, float]:
        raise NotImplementedError

    def _eval_step(self, batch) -> float:
        raise NotImplementedError

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def close(self):
        self.engine.destroy()
        if self.stats_logger is not None:
            self.stats_logger.close()
        self.profiling.close()

    def train(self, max_steps: int | None = None, step_callback=None):
        cfg = self.config
        total = cfg.total_train_steps or self.ft_spec.total_train_steps
        if max_steps is not None:
            total = min(total, max_steps)
        info = self.recover.load(self.engine, self.saver, self.evaluator, self.stats_logger, self.train_loader)
        start = info.last_step_info.global_step + 1 if info is not None else 0
        spe = self.ft_spec.steps_per_epoch
        step = 0
        # this loop replays the epochs from the start and skips the steps that were already taken, so the loader
        # starts over too (its restored position would otherwise be skipped a second time)
        self.train_loader.load_state_dict({"epoch": 0, "position": 0})
        for epoch in range(cfg.total_train_epochs):
            self.train_loader.set_epoch(epoch)
            for epoch_step, items in enumerate(self.train_loader):
                if step < start:
                    step += 1
                    continue
                if step >= total:
                    return
                batch = self.collate(items)
                with self.profiling.step(step), stats_tracker.record_timing("train_step"):
                    st = self._train_step(batch)
                self.engine.set_version(step + 1)
                with stats_tracker.record_timing("save"):
                    self.saver.save(self.engine, epoch, epoch_step, step, tokenizer=self.tokenizer,
                                    processor=self.processor)
                self.recover.dump(self.engine, StepInfo(epoch, epoch_step, step, spe), self.saver, self.evaluator,
                                  self.stats_logger, self.train_loader)
                if self.valid_loader is not None:
                    self.evaluator.evaluate(self.evaluate, epoch, epoch_step, step)
                stats = self.engine.export_stats()
                stats.update({f"step/{k}": v for k, v in st.items()})
                if self.stats_logger is not None:
                    self.stats_logger.commit(epoch, epoch_step, step, stats)
                if step_callback is not None:
                    step_callback(step, stats)
                step += 1

    def evaluate(self):
        losses = [self._eval_step(self.collate(items)) for items in self.valid_loader]
        if losses:
            stats_tracker.get("eval").scalar(loss=sum(losses) / len(losses))


class SFTTrainer(_SLTrainer):
    collate = staticmethod(collate_sft)

    def _make_wrapper(self, actor_cfg):
        return LMEngine(self.engine)

    def _train_step(self, batch):
        return self.wrapper.train_lm(batch)

    def _eval_step(self, batch):
        return self.wrapper.evaluate_lm(batch)


class RWTrainer(_SLTrainer):
    collate = staticmethod(collate_pairs)

    def __init__(self, config: RWConfig, train_dataset, valid_dataset=None, tokenizer=None):
        cfg = config.actor if getattr(config, "model", None) is None else config.model
        cfg.is_critic = True
        cfg.mb_spec.granularity = 2
        super().__init__(config, train_dataset, valid_dataset, tokenizer)

    def _make_wrapper(self, actor_cfg):
        return RWEngine(self.engine)

    def _train_step(self, batch):
        return self.wrapper.train_rw(batch)

    def _eval_step(self, batch):
        return self.wrapper.evaluate_rw(batch)


class DPOTrainer(_SLTrainer):
    collate = staticmethod(collate_pairs)

    def _make_wrapper(self, actor_cfg):
        ref = None
        if self.config.ref is not None:
            ref = B200TrainEngine(self.config.ref)
            ref.create_process_group(self.alloc.parallel)
            ref.initialize(None, self.ft_spec, seed=self.config.seed)
        self.ref_engine = ref
        return DPOEngine(actor_cfg, self.engine, ref)

    def _train_step(self, batch):
        return self.wrapper.train_dpo(batch)

    def _eval_step(self, batch):
        return self.wrapper.evaluate_dpo(batch)
