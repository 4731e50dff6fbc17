"""GSM8K reinforcement learning (GRPO / PPO and every variant selected by the YAML).

    python -m areal_b200.infra.launcher.local examples/math/gsm8k_rl.py --config examples/math/gsm8k_grpo.yaml \
        experiment_name=gsm8k trial_name=run0 actor.path=/models/Qwen3-1.7B train_dataset.path=/data/gsm8k

The launcher starts one rank per GPU of the allocation (`rollout.backend` + `actor.backend`); this
script runs on every rank.
"""
import sys

from areal_b200.api.cli_args import GRPOConfig, load_expr_config
from areal_b200.dataset import get_custom_dataset
from areal_b200.trainer.rl_trainer import PPOTrainer
from areal_b200.utils.hf_io import load_hf_tokenizer


def main(argv):
    config, _ = load_expr_config(argv, GRPOConfig)
    tokenizer = load_hf_tokenizer(config.tokenizer_path or config.actor.path)
    train = get_custom_dataset(path=config.train_dataset.path, type=config.train_dataset.type, split="train",
                               tokenizer=tokenizer, max_length=config.train_dataset.max_length)
    valid = None
    if config.valid_dataset is not None:
        valid = get_custom_dataset(path=config.valid_dataset.path, type=config.valid_dataset.type, split="test",
                                   tokenizer=tokenizer, max_length=config.valid_dataset.max_length)
    workflow_kwargs = dict(reward_fn="areal_b200.reward.gsm8k.gsm8k_reward_fn", gconfig=config.gconfig,
                           tokenizer=tokenizer, enable_thinking=False)
    eval_kwargs = dict(workflow_kwargs, gconfig=(config.eval_gconfig or config.gconfig).new(temperature=0.6))
    with PPOTrainer(config, train, valid, tokenizer=tokenizer) as trainer:
        trainer.train(workflow="areal_b200.workflow.rlvr.RLVRWorkflow", workflow_kwargs=workflow_kwargs,
                      eval_workflow="areal_b200.workflow.rlvr.RLVRWorkflow", eval_workflow_kwargs=eval_kwargs)


if __name__ == "__main__":
    main(sys.argv[1:])
