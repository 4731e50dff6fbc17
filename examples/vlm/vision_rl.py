"""GRPO on vision-language prompts (clevr_count_70k, geometry3k, virl39k) with Qwen2.5-VL.

    python -m areal_b200.infra.launcher.local examples/vlm/vision_rl.py \
        --config examples/vlm/clevr_count_70k_grpo.yaml actor.path=/models/Qwen2.5-VL-3B-Instruct \
        train_dataset.path=/data/clevr_count_70k

The reward function follows the dataset named in ``train_dataset.path``.
"""
import sys

from areal_b200.api.cli_args import GRPOConfig, load_expr_config
from areal_b200.dataset import get_custom_dataset
from areal_b200.trainer.rl_trainer import PPOTrainer
from areal_b200.utils.hf_io import load_hf_processor_and_tokenizer

REWARDS = {"clevr_count_70k": "areal_b200.reward.clevr_count_70k.clevr_count_70k_reward_fn",
           "geometry3k": "areal_b200.reward.geometry3k.geometry3k_reward_fn",
           "virl39k": "areal_b200.reward.geometry3k.geometry3k_reward_fn"}


def main(argv):
    config, _ = load_expr_config(argv, GRPOConfig)
    processor, tokenizer = load_hf_processor_and_tokenizer(config.tokenizer_path or config.actor.path)
    train = get_custom_dataset(path=config.train_dataset.path, type="rl", split="train", tokenizer=tokenizer,
                               processor=processor, max_length=config.train_dataset.max_length)
    valid = get_custom_dataset(path=config.valid_dataset.path, type="rl", split="test", tokenizer=tokenizer,
                               processor=processor) if config.valid_dataset is not None else None
    reward = next(fn for name, fn in REWARDS.items() if name in config.train_dataset.path.lower())
    workflow_kwargs = dict(reward_fn=reward, gconfig=config.gconfig, tokenizer=tokenizer, processor=processor,
                           enable_thinking=False)
    eval_kwargs = dict(workflow_kwargs, gconfig=(config.eval_gconfig or config.gconfig).new(temperature=0.6))
    wf = "areal_b200.workflow.vision_rlvr.VisionRLVRWorkflow"
    with PPOTrainer(config, train, valid, tokenizer=tokenizer, processor=processor) as trainer:
        trainer.train(workflow=wf, workflow_kwargs=workflow_kwargs, eval_workflow=wf, eval_workflow_kwargs=eval_kwargs)


if __name__ == "__main__":
    main(sys.argv[1:])
