"""GSM8K with agent code on the OpenAI chat-completions protocol: the agent (single turn, multi-turn
with retry feedback, or calculator tools) runs inside the rollout workers against an engine-bound
client, every completion it requests becomes a training sample, and its return value is the reward.

    python -m areal_b200.infra.launcher.local examples/openai_agent/gsm8k_agent_rl.py \
        --config examples/math/gsm8k_grpo.yaml experiment_name=gsm8k-agent agent=multi_turn

Agents written against a ``base_url`` (any SDK) run the same way with ``mode="online"`` and the proxy
server of ``areal_b200.openai.proxy.proxy_rollout_server``.
"""
import sys

from areal_b200.api.cli_args import GRPOConfig, load_expr_config
from areal_b200.dataset import get_custom_dataset
from areal_b200.trainer.rl_trainer import PPOTrainer
from areal_b200.utils.hf_io import load_hf_tokenizer
from areal_b200.workflow.agents import MathAgent, MathToolAgent, MultiTurnMathAgent

AGENTS = {"single": MathAgent, "multi_turn": MultiTurnMathAgent, "tool": MathToolAgent}


def pop_agent(argv: list[str], default: str = "single") -> tuple[str, list[str]]:
    """``agent=<name>`` is this script's own switch; everything else goes to the config loader."""
    kind, rest = default, []
    for a in argv:
        if a.startswith("agent="):
            kind = a.split("=", 1)[1]
        else:
            rest.append(a)
    if kind not in AGENTS:
        raise SystemExit(f"agent must be one of {sorted(AGENTS)}, got {kind!r}")
    return kind, rest


def main(argv, default_agent: str = "single"):
    kind, argv = pop_agent(list(argv), default_agent)
    config, _ = load_expr_config(argv, GRPOConfig)
    tokenizer = load_hf_tokenizer(config.tokenizer_path or config.actor.path)
    train = get_custom_dataset(path=config.train_dataset.path, type="rl", split="train", tokenizer=tokenizer,
                               max_length=config.train_dataset.max_length)
    sampling = dict(temperature=config.gconfig.temperature, top_p=config.gconfig.top_p,
                    max_completion_tokens=config.gconfig.max_new_tokens)
    agent = AGENTS[kind](**sampling) if kind == "single" else AGENTS[kind](max_turns=4, **sampling)
    with PPOTrainer(config, train, None, tokenizer=tokenizer) as trainer:
        trainer.train(workflow="areal_b200.openai.proxy.workflow.OpenAIProxyWorkflow",
                      workflow_kwargs=dict(agent=agent, tokenizer=tokenizer, gconfig=config.gconfig, mode="inline",
                                           turn_discount=0.9, export_style="individual"))


if __name__ == "__main__":
    main(sys.argv[1:])
