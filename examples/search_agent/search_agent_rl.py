"""Question answering with a search tool (ReAct loop over `search` / `visit`), trained with GRPO: every
completion of an episode is a training sample and the final answer's F1 against the gold answers is the
reward, shared with the earlier tool-calling turns through the turn discount.

    python -m areal_b200.infra.launcher.local examples/search_agent/search_agent_rl.py \
        --config examples/search_agent/search_agent_grpo.yaml corpus=/data/wiki_passages.jsonl

`corpus=<file.jsonl>` serves retrieval from an in-process BM25 index; `search_url=http://host:port` uses a
retrieval service instead (`/search`, `/visit`).
"""
import sys

from areal_b200.api.cli_args import GRPOConfig, load_expr_config
from areal_b200.dataset import get_custom_dataset
from areal_b200.trainer.rl_trainer import PPOTrainer
from areal_b200.utils.hf_io import load_hf_tokenizer
from areal_b200.workflow.agents import HttpSearch, LocalCorpus, ReActSearchAgent


def pop_switches(argv: list[str]) -> tuple[dict[str, str], list[str]]:
    """This script's own `key=value` switches; the rest goes to the config loader."""
    mine, rest = {}, []
    for a in argv:
        k, _, v = a.partition("=")
        if k in ("corpus", "search_url", "max_turns", "metric"):
            mine[k] = v
        else:
            rest.append(a)
    return mine, rest


def make_backend(switches: dict[str, str]):
    if "search_url" in switches:
        return HttpSearch(switches["search_url"])
    if "corpus" in switches:
        return LocalCorpus.from_jsonl(switches["corpus"])
    raise SystemExit("give corpus=<passages.jsonl> or search_url=<http://host:port>")


def main(argv):
    switches, argv = pop_switches(list(argv))
    config, _ = load_expr_config(argv, GRPOConfig)
    tokenizer = load_hf_tokenizer(config.tokenizer_path or config.actor.path)
    train = get_custom_dataset(path=config.train_dataset.path, type="rl", split="train", tokenizer=tokenizer,
                               max_length=config.train_dataset.max_length)
    agent = ReActSearchAgent(make_backend(switches), max_turns=int(switches.get("max_turns", 6)),
                             metric=switches.get("metric", "f1"), temperature=config.gconfig.temperature,
                             top_p=config.gconfig.top_p, max_completion_tokens=config.gconfig.max_new_tokens)
    with PPOTrainer(config, train, None, tokenizer=tokenizer) as trainer:
        trainer.train(workflow="areal_b200.openai.proxy.workflow.OpenAIProxyWorkflow",
                      workflow_kwargs=dict(agent=agent, tokenizer=tokenizer, gconfig=config.gconfig, mode="inline",
                                           turn_discount=0.9, export_style="individual"))


if __name__ == "__main__":
    main(sys.argv[1:])
