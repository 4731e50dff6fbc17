"""Terminal tasks with GRPO: the policy works in a per-episode shell workspace (`bash`, `write_file`,
`read_file` tools) and is rewarded by the fraction of the task's check commands that pass afterwards.

    python -m areal_b200.infra.launcher.local examples/terminal_bench/terminal_agent_rl.py \
        --config examples/terminal_bench/terminal_agent_grpo.yaml

Agent episodes block on subprocesses, so the workflow runs them in worker threads (`mode="subproc"`).
"""
import sys

from areal_b200.api.cli_args import GRPOConfig, load_expr_config
from areal_b200.dataset import get_custom_dataset
from areal_b200.trainer.rl_trainer import PPOTrainer
from areal_b200.utils.hf_io import load_hf_tokenizer
from areal_b200.workflow.agents import TerminalAgent


def main(argv):
    config, _ = load_expr_config(list(argv), GRPOConfig)
    tokenizer = load_hf_tokenizer(config.tokenizer_path or config.actor.path)
    train = get_custom_dataset(path=config.train_dataset.path, type="rl", split="train", tokenizer=tokenizer,
                               max_length=config.train_dataset.max_length)
    agent = TerminalAgent(max_turns=12, temperature=config.gconfig.temperature, top_p=config.gconfig.top_p,
                          max_completion_tokens=config.gconfig.max_new_tokens)
    with PPOTrainer(config, train, None, tokenizer=tokenizer) as trainer:
        trainer.train(workflow="areal_b200.openai.proxy.workflow.OpenAIProxyWorkflow",
                      workflow_kwargs=dict(agent=agent, tokenizer=tokenizer, gconfig=config.gconfig, mode="subproc",
                                           turn_discount=0.95, export_style="individual"))


if __name__ == "__main__":
    main(sys.argv[1:])
