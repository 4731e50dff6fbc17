"""PPO / GRPO trainer: asynchronous RL main loop.

    with PPOTrainer(config, train_dataset, valid_dataset) as trainer:
        trainer.train(workflow="areal_b200.workflow.rlvr.RLVRWorkflow",
                      workflow_kwargs=dict(reward_fn=..., gconfig=config.gconfig, tokenizer=tok))

Every rank runs this script (SPMD). The allocation strings decide the roles:

* ``rollout.backend = native:dA`` and ``actor.backend = fsdp:dB`` with ``A + B ==
  world`` – disaggregated: the first A ranks generate, the last B ranks train;
  trajectories and control go over gloo, weights over NVLink peer memory;
* ``A == B == world`` (or a single process) – colocated: every rank owns both a
  rollout engine and a trainer shard on the same GPU; generation runs in a
  background thread / CUDA stream while the trainer consumes the previous
  batches.

One step: wait for a batch that is at most ``max_head_offpolicyness`` versions
stale → (critic values, reference / teacher logprobs) → recompute proximal
logprobs → advantages → ``ppo_update`` → pause rollout, push weights, bump
version, resume → save / recover / evaluate / log. Mirrors the reference loop
(areal/trainer/rl_trainer.py:105-824).
"""

from __future__ import annotations

import os
import time
from typing import Any

import torch
import torch.distributed as dist

from ..api.alloc_mode import ModelAllocation
from ..api.cli_args import PPOConfig, get_log_path, save_config
from ..api.io_struct import FinetuneSpec, StepInfo, WeightUpdateMeta
from ..engine.rollout_engine import NativeRolloutEngine
from ..engine.train_engine import B200TrainEngine
from ..infra.dist_rollout import (DisaggTopology, RemoteRolloutClient, RolloutServer,
                                  exchange_weight_buffers)
from ..utils import logging, seeding, stats_tracker
from ..utils.evaluator import Evaluator
from ..utils.recover import RecoverHandler
from ..utils.saver import Saver
from ..utils.stats_logger import StatsLogger
from .ppo.actor import PPOActor
from .ppo.critic import PPOCritic

logger = logging.getLogger("PPOTrainer")


# the loader lives in utils/dataloader.py (mid-epoch state, exact evaluation split); the old private name stays
from ..utils.dataloader import StatefulListLoader as _ListLoader  # noqa: E402


class PPOTrainer:
    def __new__(cls, config: PPOConfig, *args, **kwargs):
        # `scheduler.type` set and no torchrun environment: this process is the controller of a
        # single-controller run and the engines live in scheduler workers (trainer/controller_mode.py)
        if cls is PPOTrainer and getattr(config.scheduler, "type", None) and "RANK" not in os.environ:
            from .controller_mode import ControllerPPOTrainer

            return ControllerPPOTrainer(config, *args, **kwargs)
        return super().__new__(cls)

    def __init__(self, config: PPOConfig, train_dataset, valid_dataset=None, tokenizer=None, processor=None):
        self.tokenizer = tokenizer
        self.processor = processor  # vision-language models: saved next to the weights
        self.config = config
        self.train_dataset, self.valid_dataset = train_dataset, valid_dataset
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
        self.actor_alloc = ModelAllocation.from_str(config.actor.backend)
        self.rollout_alloc = ModelAllocation.from_str(config.rollout.backend)
        n_train, n_gen = self.actor_alloc.world_size, self.rollout_alloc.world_size
        # External rollout servers (this repo's HTTP server on other nodes, SGLang, vLLM): every rank of
        # this job trains, generation goes over HTTP and weights travel through a checkpoint directory.
        self.external_rollout = (self.rollout_alloc.backend in ("sglang", "vllm")
                                 or bool(os.environ.get("AREAL_LLM_SERVER_ADDRS")))
        if self.external_rollout:
            n_gen = 0
        self.colocated = not self.external_rollout and (self.world == 1 or (n_train == self.world and n_gen == self.world))
        if not self.colocated and n_train + n_gen != self.world:
            raise ValueError(f"allocation {config.rollout.backend}+{config.actor.backend} needs "
                             f"{n_train + n_gen} ranks, world size is {self.world}")
        ps_ = self.actor_alloc.parallel
        replica = ps_.tp_size * ps_.cp_size  # ranks of one replica inside a pipeline stage (tp innermost, then sp)
        self.topo = None if (self.colocated or self.external_rollout) else DisaggTopology(
            n_gen, n_train, replica_size=replica, n_replicas=max(n_train // (replica * ps_.pp_size), 1))
        self.is_trainer = self.colocated or self.external_rollout or not self.topo.is_rollout
        self.is_rollout = not self.external_rollout and (self.colocated or self.topo.is_rollout)
        train_ranks = list(range(self.world)) if self.topo is None else self.topo.train_ranks
        dp = len(train_ranks)
        bs = config.train_dataset.batch_size
        self.ft_spec = FinetuneSpec(total_train_epochs=config.total_train_epochs,
                                    dataset_size=len(train_dataset), train_batch_size=bs)
        self.per_rank_bs = max(bs // dp, 1)
        # every role takes part in group creation (collective)
        self.actor_engine = B200TrainEngine(config.actor) if self.is_trainer else None
        self.critic_engine = None
        self.teacher_engine = None
        self.teacher = None
        self.ref_engine = None
        helper = self.actor_engine or B200TrainEngine(config.actor)
        helper.create_process_group(self.actor_alloc.parallel, ranks=train_ranks)
        self.train_cpu_group = helper.cpu_group
        shared = (helper.data_parallel_group, helper.cpu_group)
        self.rollout = None
        self.rollout_client = None
        if self.is_rollout:
            rcfg = config.rollout
            rcfg.consumer_batch_size = bs
            self.rollout = NativeRolloutEngine(rcfg)
            n_gen_eff = self.world if self.colocated else n_gen
            self.rollout.initialize(train_data_parallel_size=n_gen_eff)
        if self.is_trainer:
            self.actor_engine.initialize(None, self.ft_spec, seed=config.seed)
            if config.critic is not None:
                self.critic_engine = B200TrainEngine(config.critic)
                self.critic_engine.create_process_group(self.actor_alloc.parallel, ranks=train_ranks, groups=shared)
                self.critic_engine.initialize(None, self.ft_spec, seed=config.seed + 1)
            if getattr(config, "teacher", None) is not None:
                # distillation: a frozen teacher scores every batch; the actor's loss mixes the RL term with
                # the reverse-KL term towards it (TeacherConfig.rl_loss_weight / distill_loss_weight)
                config.teacher.optimizer = None
                self.teacher_engine = B200TrainEngine(config.teacher)
                self.teacher_engine.create_process_group(self.actor_alloc.parallel, ranks=train_ranks, groups=shared)
                self.teacher_engine.initialize(None, self.ft_spec, seed=config.seed + 2)
            if config.ref is not None and config.actor.kl_ctl != 0.0:
                self.ref_engine = B200TrainEngine(config.ref)
                self.ref_engine.create_process_group(self.actor_alloc.parallel, ranks=train_ranks, groups=shared)
                self.ref_engine.initialize(None, self.ft_spec, seed=config.seed)
        if self.external_rollout:
            from ..infra.remote_inf_engine import RemoteInfEngine

            rcfg = config.rollout
            rcfg.consumer_batch_size = bs
            self.rollout_client = RemoteInfEngine(rcfg).initialize(train_data_parallel_size=dp)
            self.weight_meta = WeightUpdateMeta(type="disk", path=os.path.join(
                config.cluster.fileroot, "weight_update", str(config.experiment_name), str(config.trial_name)))
        elif self.colocated:
            self.rollout_client = self.rollout
            self.weight_meta = WeightUpdateMeta.from_p2p()
            ps = self.actor_alloc.parallel
            if ps.tp_size * ps.pp_size * ps.ep_size > 1:
                self._connect_colocated_model_parallel(use_cuda)
        else:
            dev = torch.cuda.current_device() if use_cuda else 0
            ptrs = exchange_weight_buffers(self.topo, self.rollout, dev)
            if self.is_trainer:
                # pause / resume barriers span EVERY trainer rank: tensor- and pipeline-parallel peers push
                # their shards too and must not write before the rollout engines have paused
                self.rollout_client = RemoteRolloutClient(self.topo, ptrs, self.actor_engine._all_cpu_group)
            self.weight_meta = WeightUpdateMeta.from_p2p()
        if self.is_trainer:
            self.actor_engine.connect_engine(self.rollout_client, self.weight_meta)
            self.actor = PPOActor(config.actor, self.actor_engine)
            self.critic = PPOCritic(config.critic, self.critic_engine) if self.critic_engine else None
            self.ref = PPOActor(config.ref, self.ref_engine) if self.ref_engine else None
            self.teacher = PPOActor(config.teacher, self.teacher_engine) if self.teacher_engine else None
            if self.teacher is not None:
                self.actor.distill_weights = (float(config.teacher.rl_loss_weight),
                                              float(config.teacher.distill_loss_weight))
        self.saver = Saver(config.saver, self.ft_spec)
        self.evaluator = Evaluator(config.evaluator, self.ft_spec)
        self.recover = RecoverHandler(config.recover, self.ft_spec)
        self.stats_logger = StatsLogger(config, self.ft_spec) if self.rank == train_ranks[0] else None
        local_gen = self.colocated or self.external_rollout  # this rank asks for its own share of every batch
        gen_rank = self.rank if local_gen else (self.rank if self.is_rollout else 0)
        gen_world = self.world if local_gen else n_gen
        self.dataloader = _ListLoader(train_dataset, self.per_rank_bs if local_gen else max(bs // gen_world, 1),
                                      config.train_dataset.shuffle, config.seed, gen_rank, gen_world)
        self.step_times: list[float] = []
        self.trained_tokens = 0
        from ..utils.step_profiling import StepProfiling

        self.profiling = StepProfiling(config, self.rank, "trainer" if self.is_trainer else "rollout")
        if self.rank == train_ranks[0]:
            try:
                save_config(config, get_log_path(config))
            except Exception as e:
                logger.warning(f"could not save the config: {e}")

    def _connect_colocated_model_parallel(self, use_cuda: bool):
        """Colocated layout with a tensor- / pipeline- / expert-parallel trainer: every rank's rollout engine
        holds the whole model, every trainer rank a shard. The ranks exchange handles of their rollout weight
        buffers so that each trainer rank can store its share of the re-sharding plan into all of them."""
        if not use_cuda:
            raise NotImplementedError("a colocated model-parallel trainer pushes weights through CUDA peer memory")
        from ..infra.weight_plan import WeightPusher, rollout_layout
        from ..parallel.symm_mem import open_ipc_handle

        flat = self.rollout.flat
        handles = [None] * self.world
        group = self.actor_engine._all_cpu_group
        dist.all_gather_object(handles, flat.param_buf.ipc_handle(), group=group)
        dev = torch.cuda.current_device()
        ptrs = [flat.flat.data_ptr() if r == self.rank else open_ipc_handle(h, dev) for r, h in enumerate(handles)]
        self.rollout.weight_pusher = (WeightPusher(self.actor_engine, ptrs, rollout_layout(flat)), group)

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def close(self):
        if self.rollout_client is not None and self.external_rollout:
            self.rollout_client.destroy()
        elif self.rollout_client is not None and not self.colocated:
            self.rollout_client.stop()
        if self.rollout is not None:
            self.rollout.destroy()
        for e in (self.actor_engine, self.critic_engine, self.ref_engine, getattr(self, "teacher_engine", None)):
            if e is not None:
                e.destroy()
        if self.stats_logger is not None:
            self.stats_logger.close()
        self.profiling.close()

    def _next_batch(self, workflow, workflow_kwargs, group):
        """The next training batch of this rank. Under tensor / sequence / pipeline parallelism only
        the head of each data-parallel replica talks to the rollout side; the other ranks of the
        replica receive the same batch over their model-parallel group."""
        cfg = self.config
        eng = self.actor_engine
        mp = getattr(eng, "context_and_model_parallel_group", None)
        if mp is None or dist.get_world_size(mp) == 1:
            batch = self.rollout_client.prepare_batch(self.dataloader, workflow, workflow_kwargs,
                                                      group_size=group, dynamic_bs=cfg.dynamic_bs)
            if self.colocated and eng.mesh is None and eng.world_size > 1 and not cfg.dynamic_bs \
                    and os.environ.get("AREAL_B200_BALANCE_DP", "1") == "1":
                # every rank rolled out its own prompts; response lengths differ a lot, and the step takes as long
                # as the most loaded rank: deal the pooled samples out again by token count (sample groups intact)
                from ..infra.dist_rollout import redistribute_trajectories

                batch = redistribute_trajectories(batch, eng.cpu_group, granularity=group).data
            return batch
        box = [None]
        if eng.is_data_parallel_head():
            box[0] = self.rollout_client.prepare_batch(self.dataloader, workflow, workflow_kwargs,
                                                       group_size=group, dynamic_bs=cfg.dynamic_bs)
        dist.broadcast_object_list(box, src=eng.current_data_parallel_head(), group=mp)
        return box[0]

    # -------------------------------------------------------------------- train
    def train(self, workflow, workflow_kwargs: dict | None = None, eval_workflow=None,
              eval_workflow_kwargs: dict | None = None, max_steps: int | None = None,
              step_callback=None):
        cfg = self.config
        total = cfg.total_train_steps or self.ft_spec.total_train_steps
        if max_steps is not None:
            total = min(total, max_steps)
        group = cfg.gconfig.n_samples
        if not self.is_trainer:
            # rollout-only rank of a disaggregated run: produce batches until told to stop
            server = RolloutServer(self.topo, self.rollout)
            if eval_workflow is not None and self.valid_dataset is not None:
                gi, ng = self.topo.gen_ranks.index(self.topo.rank), len(self.topo.gen_ranks)
                server.set_eval([self.valid_dataset[i] for i in range(gi, len(self.valid_dataset), ng)],
                                eval_workflow, eval_workflow_kwargs)
            server.serve(self.dataloader, workflow, workflow_kwargs, group_size=group, n_steps=total)
            server.wait_stop(timeout=600)
            return
        start = 0
        info = self.recover.load(self.actor_engine, self.saver, self.evaluator, self.stats_logger,
                                 self.dataloader, self.rollout if self.colocated else None, self.weight_meta)
        if info is not None:
            start = info.last_step_info.global_step + 1
        else:
            # both sides start from identical weights and version 0
            self.actor_engine.update_weights(self.weight_meta.with_version(0))
        steps_per_epoch = self.ft_spec.steps_per_epoch
        for global_step in range(start, total):
            t_step = time.perf_counter()
            epoch, epoch_step = divmod(global_step, steps_per_epoch)
            with self.profiling.step(global_step):
                with stats_tracker.record_timing("rollout"):
                    batch = self._next_batch(workflow, workflow_kwargs, group)
                stats = self.train_step(batch, global_step)
            self.step_times.append(time.perf_counter() - t_step)
            with stats_tracker.record_timing("save"):
                self.saver.save(self.actor_engine, epoch, epoch_step, global_step, tokenizer=self.tokenizer,
                                processor=self.processor)
            with stats_tracker.record_timing("checkpoint_for_recover"):
                self.recover.dump(self.actor_engine, StepInfo(epoch, epoch_step, global_step, steps_per_epoch),
                                  self.saver, self.evaluator, self.stats_logger, self.dataloader)
            if eval_workflow is not None and self.valid_dataset is not None:
                self.evaluator.evaluate(lambda: self._evaluate(eval_workflow, eval_workflow_kwargs),
                                        epoch, epoch_step, global_step)
            exported = self.actor_engine.export_stats()
            exported.update(stats)
            if self.stats_logger is not None:
                self.stats_logger.commit(epoch, epoch_step, global_step, exported)
            if step_callback is not None:
                step_callback(global_step, exported)

    def train_step(self, batch: dict[str, Any], global_step: int) -> dict[str, float]:
        """Everything between receiving a rollout batch and resuming generation."""
        cfg = self.config
        actor = self.actor
        if self.critic is not None:
            with stats_tracker.record_timing("critic_values"):
                batch["values"] = self.critic.compute_values(batch)
        if self.ref is not None:
            with stats_tracker.record_timing("ref_logp"):
                batch["ref_logp"] = self.ref.compute_logp(batch)
        if getattr(self, "teacher", None) is not None:
            with stats_tracker.record_timing("teacher_logp"):
                batch["teacher_logp"] = self.teacher.compute_logp(batch)
        if cfg.actor.should_compute_prox_logp():
            with stats_tracker.record_timing("recompute_logp"):
                batch["prox_logp"] = actor.compute_logp(batch)
        with stats_tracker.record_timing("compute_advantage"):
            adv_batch = actor.compute_advantages(batch)
        with stats_tracker.record_timing("train_step"):
            train_stats = actor.ppo_update(adv_batch)
        if self.critic is not None:
            with stats_tracker.record_timing("critic_train_step"):
                self.critic.ppo_update(adv_batch)
        n_tok = int(batch["attention_mask"].sum())
        self.trained_tokens += n_tok
        new_version = global_step + 1
        with stats_tracker.record_timing("update_weights"):
            self.rollout_client.pause()
            sync_s = self.actor_engine.update_weights(self.weight_meta.with_version(new_version))
            self.actor_engine.set_version(new_version)
            if self.critic_engine is not None:
                self.critic_engine.set_version(new_version)
            self.rollout_client.resume()
        n_resp = int(batch["loss_mask"].sum()) if "loss_mask" in batch else n_tok
        out = {"step/trained_tokens": float(n_tok), "step/response_tokens": float(n_resp),
               "step/weight_sync_s": float(sync_s),
               "step/loss": float(train_stats[-1].get("loss", 0.0)),
               "step/grad_norm": float(train_stats[-1].get("grad_norm", 0.0))}
        return out

    def _evaluate(self, workflow, workflow_kwargs):
        if not self.colocated:
            # the rollout ranks hold the validation set and the evaluation workflow (``RolloutServer.set_eval``)
            total, n = self.rollout_client.evaluate()
            if n:
                stats_tracker.get("eval").scalar(reward=total / n)
            return
        items = [self.valid_dataset[i] for i in range(self.rank, len(self.valid_dataset), self.world)]
        batch = self.rollout.rollout_batch(items, workflow, workflow_kwargs, is_eval=True)
        if batch:
            stats_tracker.get("eval").scalar(reward=float(batch["rewards"].float().mean()))
