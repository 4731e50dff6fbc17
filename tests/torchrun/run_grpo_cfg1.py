"""Worker for the two-rank CPU/gloo GRPO step (tiny Qwen2 architecture, fp32, seed 0):
one synchronous rollout → train → weight-update step per rank pair, checked for
cross-rank consistency. Launched by tests/test_e2e_grpo_cpu.py through torchrun."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from areal_b200.api.cli_args import (GenerationHyperparameters, GRPOConfig, InferenceEngineConfig,  # noqa: E402
                                     MicroBatchSpec, NativeRolloutConfig, NormConfig, OptimizerConfig,
                                     PPOActorConfig, _propagate_names)
from areal_b200.trainer.rl_trainer import PPOTrainer  # noqa: E402
from areal_b200.workflow.rlvr import RLVRWorkflow  # noqa: E402


def reward_fn(prompt, completion, prompt_ids, completion_ids, **kw):
    even = sum(1 for t in completion_ids if t % 2 == 0)
    return 1.0 if even > len(completion_ids) / 2 else 0.0


def main(out_path: str, mode: str):
    torch.set_num_threads(2)
    world = int(os.environ["WORLD_SIZE"])
    preset = os.environ.get("AREAL_B200_TEST_PRESET", "tiny-qwen2")
    cfg = GRPOConfig(experiment_name="cfg1", trial_name=mode)
    cfg.seed = 0
    cfg.cluster.fileroot = os.environ.get("AREAL_B200_FILEROOT", "/tmp/areal_b200_test")
    cfg.train_dataset.batch_size = 16
    cfg.train_dataset.shuffle = False
    cfg.gconfig = GenerationHyperparameters(n_samples=4, max_new_tokens=32, temperature=1.0, ignore_eos=True)
    n_gen, n_train = (world, world) if mode == "colocated" else (world // 2, world // 2)
    cfg.actor = PPOActorConfig(backend=f"fsdp:d{n_train}", model_preset=preset, init_from_scratch=True,
                               optimizer=OptimizerConfig(lr=1e-3, warmup_steps_proportion=0.0),
                               mb_spec=MicroBatchSpec(max_tokens_per_mb=1024), ppo_n_minibatches=1,
                               reward_norm=NormConfig(mean_level="group", std_level="group", group_size=4),
                               kl_ctl=0.0, use_decoupled_loss=True, recompute_logprob=True)
    cfg.rollout = InferenceEngineConfig(backend=f"native:d{n_gen}", max_head_offpolicyness=0,
                                        max_concurrent_rollouts=64,
                                        native=NativeRolloutConfig(model_preset=preset, context_length=128,
                                                                   max_num_seqs=32, max_num_batched_tokens=2048,
                                                                   num_kv_blocks=256, seed=0))
    _propagate_names(cfg)
    g = torch.Generator().manual_seed(0)
    ds = []
    for _ in range(16 * 3):
        L = int(torch.randint(32, 65, (1,), generator=g))
        ds.append(dict(input_ids=torch.randint(0, 1024, (L,), generator=g).tolist()))
    valid = [dict(input_ids=torch.randint(0, 1024, (24,), generator=g).tolist()) for _ in range(6)]
    cfg.evaluator.freq_steps = 1
    seen = []
    wf_kwargs = dict(reward_fn=reward_fn, gconfig=cfg.gconfig, reward_in_process=True)
    with PPOTrainer(cfg, ds, valid) as tr:
        tr.train(workflow=RLVRWorkflow, workflow_kwargs=wf_kwargs, eval_workflow=RLVRWorkflow,
                 eval_workflow_kwargs=dict(wf_kwargs, gconfig=cfg.gconfig.new(n_samples=1, max_new_tokens=8)),
                 max_steps=2, step_callback=lambda s, st: seen.append(st))
        res = {"rank": tr.rank, "is_trainer": tr.is_trainer}
        if tr.is_trainer:
            flat = tr.actor_engine.flat.flat
            res.update(checksum=float(flat.double().sum()), absum=float(flat.double().abs().sum()),
                       version=tr.actor_engine.get_version(), steps=len(seen),
                       grad_norm=[s["step/grad_norm"] for s in seen], loss=[s["step/loss"] for s in seen],
                       tokens=[s["step/trained_tokens"] for s in seen],
                       eval_reward=[next((v for k, v in s.items() if k.startswith("eval") and k.endswith("reward")), None)
                                    for s in seen])
            if tr.colocated:
                rflat = tr.rollout.flat.flat
                differing = [n for n, p_, o, k in tr.actor_engine.flat.entries
                             if not torch.equal(rflat[o:o + k], flat[o:o + k])]
                res.update(rollout_version=tr.rollout.get_version(), differing=differing[:8],
                           rollout_matches=bool(not differing and len(tr.actor_engine.flat.entries) > 0))
        else:
            res.update(rollout_version=tr.rollout.get_version())
        with open(f"{out_path}.{tr.rank}", "w") as f:
            json.dump(res, f)
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main(sys.argv[1], sys.argv[2])
