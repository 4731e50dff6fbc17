"""Bradley-Terry reward model on HH-RLHF preference pairs.

    python -m areal_b200.infra.launcher.local examples/alignment/hhrlhf_rw.py --config examples/alignment/hhrlhf_rw.yaml
"""
import sys

from areal_b200.api.cli_args import RWConfig, load_expr_config
from areal_b200.dataset import get_custom_dataset
from areal_b200.trainer.rw_trainer import RWTrainer
from areal_b200.utils.hf_io import load_hf_tokenizer


def main(argv):
    config, _ = load_expr_config(argv, RWConfig)
    tokenizer = load_hf_tokenizer(config.tokenizer_path or config.actor.path)
    train = get_custom_dataset(path=config.train_dataset.path, type="rw", split="train", tokenizer=tokenizer,
                               max_length=config.train_dataset.max_length)
    with RWTrainer(config, train, None, tokenizer=tokenizer) as trainer:
        trainer.train()


if __name__ == "__main__":
    main(sys.argv[1:])
