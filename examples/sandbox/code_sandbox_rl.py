"""GRPO on program synthesis with an execution reward: the completion's program runs against the task's
input/output cases in the sandbox (`areal_b200.infra.sandbox.LocalSandbox`: fresh interpreter, CPU / memory /
file-size limits, empty environment, wall-clock time-out) and the reward is the fraction of cases it passes.

    python -m areal_b200.infra.launcher.local examples/sandbox/code_sandbox_rl.py \
        --config examples/sandbox/code_sandbox_grpo.yaml train_dataset.path=/data/code_tasks

The reward runs in the workflow's reward process pool, so slow programs do not stall generation.
"""
import sys

from areal_b200.api.cli_args import GRPOConfig, load_expr_config
from areal_b200.dataset import get_custom_dataset
from areal_b200.trainer.rl_trainer import PPOTrainer
from areal_b200.utils.hf_io import load_hf_tokenizer


def main(argv):
    config, _ = load_expr_config(list(argv), GRPOConfig)
    tokenizer = load_hf_tokenizer(config.tokenizer_path or config.actor.path)
    train = get_custom_dataset(path=config.train_dataset.path, type="rl", split="train", tokenizer=tokenizer,
                               max_length=config.train_dataset.max_length)
    kwargs = dict(reward_fn="areal_b200.reward.code.code_reward_fn", gconfig=config.gconfig, tokenizer=tokenizer,
                  enable_thinking=False, reward_timeout=60.0)
    with PPOTrainer(config, train, None, tokenizer=tokenizer) as trainer:
        trainer.train(workflow="areal_b200.workflow.rlvr.RLVRWorkflow", workflow_kwargs=kwargs)


if __name__ == "__main__":
    main(sys.argv[1:])
