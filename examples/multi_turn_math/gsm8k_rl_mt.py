"""Multi-turn GSM8K: the policy may retry after a wrong answer; later turns are discounted.

    python -m areal_b200.infra.launcher.local examples/multi_turn_math/gsm8k_rl_mt.py \
        --config examples/math/gsm8k_grpo.yaml experiment_name=gsm8k-mt
"""
import sys

from areal_b200.api.cli_args import GRPOConfig, load_expr_config
from areal_b200.dataset import get_custom_dataset
from areal_b200.reward.gsm8k import gsm8k_reward_fn
from areal_b200.trainer.rl_trainer import PPOTrainer
from areal_b200.utils.hf_io import load_hf_tokenizer


def main(argv):
    config, _ = load_expr_config(argv, GRPOConfig)
    tokenizer = load_hf_tokenizer(config.tokenizer_path or config.actor.path)
    train = get_custom_dataset(path=config.train_dataset.path, type="rl", split="train", tokenizer=tokenizer,
                               max_length=config.train_dataset.max_length)
    with PPOTrainer(config, train, None, tokenizer=tokenizer) as trainer:
        trainer.train(workflow="areal_b200.workflow.multi_turn.MultiTurnWorkflow",
                      workflow_kwargs=dict(reward_fn=gsm8k_reward_fn, gconfig=config.gconfig, tokenizer=tokenizer,
                                           max_turns=3, turn_discount=0.9))


if __name__ == "__main__":
    main(sys.argv[1:])
