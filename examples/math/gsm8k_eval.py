"""Evaluation only: roll out the validation set with the rollout engine and report the mean reward.

    python examples/math/gsm8k_eval.py --config examples/math/gsm8k_grpo.yaml rollout.native.model_path=/models/ckpt
"""
import sys

import torch

from areal_b200.api.cli_args import GRPOConfig, load_expr_config
from areal_b200.dataset import get_custom_dataset
from areal_b200.engine.rollout_engine import NativeRolloutEngine
from areal_b200.utils.hf_io import load_hf_tokenizer
from areal_b200.workflow.rlvr import RLVRWorkflow


def main(argv):
    config, _ = load_expr_config(argv, GRPOConfig)
    tokenizer = load_hf_tokenizer(config.tokenizer_path or config.actor.path)
    data = get_custom_dataset(path=config.valid_dataset.path, type="rl", split="test", tokenizer=tokenizer)
    engine = NativeRolloutEngine(config.rollout).initialize()
    wf = RLVRWorkflow(reward_fn="areal_b200.reward.gsm8k.gsm8k_reward_fn",
                      gconfig=(config.eval_gconfig or config.gconfig).new(n_samples=1, temperature=0.0), tokenizer=tokenizer)
    rewards = []
    bs = config.valid_dataset.batch_size
    for i in range(0, len(data), bs):
        batch = engine.rollout_batch([data[j] for j in range(i, min(i + bs, len(data)))], workflow=wf)
        rewards.append(batch["rewards"].float())
    print(f"mean reward over {sum(r.numel() for r in rewards)} samples: {torch.cat(rewards).mean():.4f}")
    engine.destroy()


if __name__ == "__main__":
    main(sys.argv[1:])
