"""Supervised fine-tuning of Qwen2.5-VL on clevr_count_70k (image + counting question → answer).

    python -m areal_b200.infra.launcher.local examples/vlm/clevr_count_70k_sft.py \
        --config examples/vlm/clevr_count_70k_sft.yaml actor.path=/models/Qwen2.5-VL-3B-Instruct \
        train_dataset.path=/data/clevr_count_70k
"""
import sys

from areal_b200.api.cli_args import SFTConfig, load_expr_config
from areal_b200.dataset import get_custom_dataset
from areal_b200.trainer.sft_trainer import SFTTrainer
from areal_b200.utils.hf_io import load_hf_processor_and_tokenizer


def main(argv):
    config, _ = load_expr_config(argv, SFTConfig)
    processor, tokenizer = load_hf_processor_and_tokenizer(config.tokenizer_path or config.actor.path)
    train = get_custom_dataset(path=config.train_dataset.path, type="sft", split="train", tokenizer=tokenizer,
                               processor=processor, max_length=config.train_dataset.max_length)
    valid = get_custom_dataset(path=config.valid_dataset.path, type="sft", split="test", tokenizer=tokenizer,
                               processor=processor, max_length=config.valid_dataset.max_length) \
        if config.valid_dataset else None
    with SFTTrainer(config, train, valid, tokenizer=tokenizer, processor=processor) as trainer:
        trainer.train()


if __name__ == "__main__":
    main(sys.argv[1:])
