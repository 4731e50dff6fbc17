"""Single-controller mode of the PPO trainer (``scheduler.type: local``): one controller process, the train
engines and rollout engines in scheduler workers (gloo ranks on CPU), batches as RTensor handles, weight
updates through a checkpoint directory. Reference: areal/trainer/rl_trainer.py:121-123,876,933-1041."""
import pytest
import torch

from areal_b200.api.cli_args import (GenerationHyperparameters, GRPOConfig, InferenceEngineConfig, MicroBatchSpec,
                                     NativeRolloutConfig, NormConfig, OptimizerConfig, PPOActorConfig,
                                     _propagate_names)
from areal_b200.infra.scheduler.exceptions import WorkerFailedError
from areal_b200.trainer.controller_mode import ControllerPPOTrainer
from areal_b200.trainer.rl_trainer import PPOTrainer


def _config(tmp_path):
    cfg = GRPOConfig(experiment_name="cfg1ctl", trial_name="t")
    cfg.seed = 0
    cfg.cluster.fileroot = str(tmp_path)
    cfg.scheduler.type = "local"
    cfg.train_dataset.batch_size = 8
    cfg.train_dataset.shuffle = False
    cfg.gconfig = GenerationHyperparameters(n_samples=4, max_new_tokens=16, temperature=1.0, ignore_eos=True)
    cfg.actor = PPOActorConfig(backend="fsdp:d2", model_preset="tiny-qwen2", init_from_scratch=True, dtype="float32",
                               optimizer=OptimizerConfig(lr=1e-3, warmup_steps_proportion=0.0),
                               mb_spec=MicroBatchSpec(max_tokens_per_mb=1024), ppo_n_minibatches=1,
                               reward_norm=NormConfig(mean_level="group", std_level="group", group_size=4),
                               kl_ctl=0.0, use_decoupled_loss=True, recompute_logprob=True)
    cfg.rollout = InferenceEngineConfig(backend="native:d2", max_head_offpolicyness=0, max_concurrent_rollouts=32,
                                        native=NativeRolloutConfig(model_preset="tiny-qwen2", context_length=128,
                                                                   max_num_seqs=32, max_num_batched_tokens=2048,
                                                                   num_kv_blocks=256, seed=0, dtype="float32"))
    _propagate_names(cfg)
    g = torch.Generator().manual_seed(0)
    ds = [dict(input_ids=torch.randint(0, 1024, (int(torch.randint(16, 33, (1,), generator=g)),), generator=g).tolist())
          for _ in range(8 * 4)]
    return cfg, ds


def test_grpo_steps_in_controller_mode_match_a_local_engine(tmp_path):
    cfg, ds = _config(tmp_path)
    seen, batches, sums = [], [], []
    wf_kwargs = dict(reward_fn="tests.torchrun.run_grpo_cfg1.reward_fn", gconfig=cfg.gconfig, reward_in_process=True)
    with PPOTrainer(cfg, ds) as tr:
        assert isinstance(tr, ControllerPPOTrainer)
        assert len(tr.actor.workers) == 2 and len(tr.rollout.workers) == 2

        def on_step(step, stats):
            seen.append(stats)
            batches.append({k: (v.clone() if torch.is_tensor(v) else v) for k, v in tr.last_batch.items()})
            # after every step the rollout workers serve the new version and the trainer replicas agree
            assert tr.rollout.get_version() == step + 1
            sums.append([tr.scheduler.call_engine(w.id, "flat_checksum", "actor") for w in tr.actor.workers])

        tr.train(workflow="areal_b200.workflow.rlvr.RLVRWorkflow", workflow_kwargs=wf_kwargs, max_steps=2,
                 step_callback=on_step)
        ft_spec = tr.ft_spec
    batch0 = batches[0]
    assert all(a == b for a, b in sums) and sums[0][0] != sums[1][0]
    assert len(seen) == 2 and all(torch.isfinite(torch.tensor(s["step/loss"])) for s in seen)
    assert batch0["input_ids"].shape[0] == 32 and set(batch0["versions"].unique().tolist()) <= {-1, 0}
    # the same first batch through an engine in this process (one rank, same seed): same gradient norm, and the
    # workers' losses (each reports its share of the global loss) add up to the local one
    from areal_b200.trainer.ppo.actor import PPOActorEngine

    cfg.actor.backend = "fsdp:d1"
    local = PPOActorEngine(cfg.actor)
    local.create_process_group()
    local.initialize(None, ft_spec, seed=cfg.seed)
    batch0.pop("prox_logp", None)
    batch0["prox_logp"] = local.compute_logp(batch0)
    st = local.ppo_update(local.compute_advantages(batch0))[-1]
    assert seen[0]["step/grad_norm"] == pytest.approx(st["grad_norm"], rel=2e-4)
    assert 2 * seen[0]["step/loss"] == pytest.approx(st["loss"], rel=2e-4, abs=1e-6)


def test_a_dead_worker_surfaces_as_worker_failed_error(tmp_path):
    cfg, ds = _config(tmp_path)
    cfg.trial_name = "kill"
    _propagate_names(cfg)
    with PPOTrainer(cfg, ds) as tr:
        info = tr.scheduler._workers["actor"][1]
        info.process.kill()
        info.process.wait(timeout=30)
        with pytest.raises(WorkerFailedError):
            tr.actor.set_version(3)
