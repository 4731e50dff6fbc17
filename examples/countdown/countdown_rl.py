"""GRPO on the Countdown numbers game (reach a target with +, -, *, / over given numbers, each used once).

    # 1. make the puzzles (offline, solvable by construction)
    python examples/countdown/countdown_rl.py --make-data /data/countdown --n-train 20000 --n-test 500
    # 2. train
    python -m areal_b200.infra.launcher.local examples/countdown/countdown_rl.py \
        --config examples/countdown/countdown_grpo.yaml actor.path=/models/Qwen2.5-3B-Instruct \
        train_dataset.path=/data/countdown valid_dataset.path=/data/countdown
"""
import argparse
import os
import sys

from areal_b200.api.cli_args import GRPOConfig, load_expr_config
from areal_b200.dataset import get_custom_dataset
from areal_b200.dataset.countdown import generate
from areal_b200.trainer.rl_trainer import PPOTrainer
from areal_b200.utils.hf_io import load_hf_tokenizer


def make_data(argv):
    ap = argparse.ArgumentParser()
    ap.add_argument("--make-data", required=True, help="output directory (must contain 'countdown' in its path)")
    ap.add_argument("--n-train", type=int, default=20000)
    ap.add_argument("--n-test", type=int, default=500)
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)
    print(generate(os.path.join(a.make_data, "train.jsonl"), a.n_train, seed=a.seed))
    print(generate(os.path.join(a.make_data, "test.jsonl"), a.n_test, seed=a.seed + 1))


def main(argv):
    if "--make-data" in argv:
        return make_data(argv)
    config, _ = load_expr_config(argv, GRPOConfig)
    tokenizer = load_hf_tokenizer(config.tokenizer_path or config.actor.path)
    train = get_custom_dataset(path=config.train_dataset.path, type="rl", split="train", tokenizer=tokenizer)
    valid = get_custom_dataset(path=config.valid_dataset.path, type="rl", split="test", tokenizer=tokenizer) \
        if config.valid_dataset is not None else None
    kwargs = dict(reward_fn="areal_b200.reward.countdown.countdown_reward_fn", gconfig=config.gconfig,
                  tokenizer=tokenizer, enable_thinking=False)
    eval_kwargs = dict(kwargs, gconfig=(config.eval_gconfig or config.gconfig).new(temperature=0.6))
    wf = "areal_b200.workflow.rlvr.RLVRWorkflow"
    with PPOTrainer(config, train, valid, tokenizer=tokenizer) as trainer:
        trainer.train(workflow=wf, workflow_kwargs=kwargs, eval_workflow=wf, eval_workflow_kwargs=eval_kwargs)


if __name__ == "__main__":
    main(sys.argv[1:])
