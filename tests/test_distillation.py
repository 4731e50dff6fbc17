"""On-policy distillation in the RL trainer: a frozen teacher scores every batch and the actor's loss
mixes the policy-gradient term with the reverse-KL term towards the teacher."""
import torch

from areal_b200.api.cli_args import (GenerationHyperparameters, GRPOConfig, InferenceEngineConfig, MicroBatchSpec,
                                     NativeRolloutConfig, NormConfig, OptimizerConfig, PPOActorConfig, TeacherConfig,
                                     _propagate_names)
from areal_b200.trainer.rl_trainer import PPOTrainer
from areal_b200.workflow.rlvr import RLVRWorkflow


def _cfg(tmp_path, rl_w, kd_w):
    cfg = GRPOConfig(experiment_name="distill", trial_name=f"t{rl_w}")
    cfg.cluster.fileroot = str(tmp_path)
    cfg.train_dataset.batch_size = 4
    cfg.train_dataset.shuffle = False
    cfg.gconfig = GenerationHyperparameters(n_samples=2, max_new_tokens=8, temperature=1.0, ignore_eos=True)
    common = dict(backend="fsdp:d1", model_preset="tiny-qwen2", init_from_scratch=True,
                  mb_spec=MicroBatchSpec(max_tokens_per_mb=1024))
    cfg.actor = PPOActorConfig(optimizer=OptimizerConfig(lr=2e-3, warmup_steps_proportion=0.0), ppo_n_minibatches=1,
                               reward_norm=NormConfig(mean_level="group", std_level="group", group_size=2),
                               kl_ctl=0.0, use_decoupled_loss=True, recompute_logprob=True, **common)
    cfg.teacher = TeacherConfig(rl_loss_weight=rl_w, distill_loss_weight=kd_w, **common)
    cfg.rollout = InferenceEngineConfig(backend="native:d1", max_head_offpolicyness=0, max_concurrent_rollouts=16,
                                        native=NativeRolloutConfig(model_preset="tiny-qwen2", context_length=128,
                                                                   max_num_seqs=8, max_num_batched_tokens=512,
                                                                   num_kv_blocks=64, seed=0, cuda_graph=False))
    _propagate_names(cfg)
    return cfg


def _run(tmp_path, rl_w, kd_w, steps=2):
    g = torch.Generator().manual_seed(0)
    ds = [dict(input_ids=torch.randint(0, 1024, (10,), generator=g).tolist()) for _ in range(16)]
    seen = []
    with PPOTrainer(_cfg(tmp_path, rl_w, kd_w), ds) as tr:
        assert tr.teacher is not None and tr.teacher_engine.optimizer is None
        assert tr.actor.distill_weights == (rl_w, kd_w)
        teacher_before = tr.teacher_engine.flat.flat.clone()
        tr.train(workflow=RLVRWorkflow, workflow_kwargs=dict(
            reward_fn=lambda p, c, pi, ci, **kw: float(sum(ci) % 2), gconfig=tr.config.gconfig, reward_in_process=True),
            max_steps=steps, step_callback=lambda s, st: seen.append(st))
        assert torch.equal(tr.teacher_engine.flat.flat, teacher_before)  # the teacher never trains
    return seen


def test_distillation_mixes_rl_and_teacher_terms(tmp_path):
    seen = _run(tmp_path / "mix", 1.0, 0.5)
    assert len(seen) == 2 and all("timeperf/teacher_logp" in s for s in seen)
    assert all(torch.isfinite(torch.tensor(s["step/loss"])) and s["step/grad_norm"] > 0 for s in seen)


def test_pure_distillation(tmp_path):
    seen = _run(tmp_path / "pure", 0.0, 1.0)
    assert len(seen) == 2 and all(s["step/grad_norm"] > 0 for s in seen)
