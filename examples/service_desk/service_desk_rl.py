"""Service-desk agent with GRPO (tau-bench style): the policy serves a simulated customer at an airline desk with
database tools and a written policy; the reward is the database's final state.

    python -m areal_b200.infra.launcher.local examples/service_desk/service_desk_rl.py \
        --config examples/service_desk/service_desk_grpo.yaml

The customer is scripted by default (`ScriptedUser`). To let another model play it, pass an OpenAI-compatible async
client as `user_client` and `user="llm"` to `ServiceDeskAgent` (its tokens are not trained on: only the agent's
completions go through the recording client).
"""
import sys

from areal_b200.api.cli_args import GRPOConfig, load_expr_config
from areal_b200.dataset import get_custom_dataset
from areal_b200.trainer.rl_trainer import PPOTrainer
from areal_b200.utils.hf_io import load_hf_tokenizer
from areal_b200.workflow.agents import ServiceDeskAgent


def main(argv):
    config, _ = load_expr_config(list(argv), GRPOConfig)
    tokenizer = load_hf_tokenizer(config.tokenizer_path or config.actor.path)
    train = get_custom_dataset(path=config.train_dataset.path, type="rl", split="train", tokenizer=tokenizer,
                               max_length=config.train_dataset.max_length)
    valid = get_custom_dataset(path=config.valid_dataset.path, type="rl", split="test", tokenizer=tokenizer) \
        if config.valid_dataset is not None and config.valid_dataset.path else None
    agent = ServiceDeskAgent(max_turns=20, temperature=config.gconfig.temperature, top_p=config.gconfig.top_p,
                             max_completion_tokens=config.gconfig.max_new_tokens)
    kwargs = dict(agent=agent, tokenizer=tokenizer, gconfig=config.gconfig, turn_discount=1.0,
                  export_style="individual")
    with PPOTrainer(config, train, valid, tokenizer=tokenizer) as trainer:
        trainer.train(workflow="areal_b200.openai.proxy.workflow.OpenAIProxyWorkflow", workflow_kwargs=kwargs,
                      eval_workflow="areal_b200.openai.proxy.workflow.OpenAIProxyWorkflow" if valid else None,
                      eval_workflow_kwargs=dict(kwargs, gconfig=config.gconfig.new(n_samples=1)) if valid else None)


if __name__ == "__main__":
    main(sys.argv[1:])
