"""Training side of online mode: rollout workers serve the OpenAI-compatible proxy, announce themselves to the
gateway and train on whatever sessions external users drive (see `external_user.py` for the user side).

    # 1. the gateway (stateless; one per job)
    python -m uvicorn --factory areal_b200.openai.proxy.proxy_gateway:create_gateway_app --port 8000
    # 2. the job
    python -m areal_b200.infra.launcher.local examples/online_proxy/online_rl.py \
        --config examples/math/gsm8k_grpo.yaml gateway=http://127.0.0.1:8000 proxy=http://127.0.0.1:8100

The dataset only paces the loop here (one item = one slot for an external episode); prompts come from the users.
"""
import sys

from areal_b200.api.cli_args import GRPOConfig, load_expr_config
from areal_b200.openai.proxy.online_agent import OnlineAgent
from areal_b200.trainer.rl_trainer import PPOTrainer
from areal_b200.utils.hf_io import load_hf_tokenizer


def pop_switches(argv):
    mine, rest = {}, []
    for a in argv:
        k, _, v = a.partition("=")
        if k in ("gateway", "proxy", "admin_key", "slots"):
            mine[k] = v
        else:
            rest.append(a)
    return mine, rest


def main(argv):
    switches, argv = pop_switches(list(argv))
    if "gateway" not in switches or "proxy" not in switches:
        raise SystemExit("give gateway=<url of the gateway> and proxy=<url this job's proxy server listens on>")
    config, _ = load_expr_config(argv, GRPOConfig)
    tokenizer = load_hf_tokenizer(config.tokenizer_path or config.actor.path)
    admin = switches.get("admin_key", "areal-admin-key")
    slots = [{"slot": i} for i in range(int(switches.get("slots", 1024)))]
    agent = OnlineAgent(switches["gateway"], worker_addr=switches["proxy"].split("//", 1)[-1], admin_api_key=admin)
    with PPOTrainer(config, slots, None, tokenizer=tokenizer) as trainer:
        trainer.train(workflow="areal_b200.openai.proxy.workflow.OpenAIProxyWorkflow",
                      workflow_kwargs=dict(agent=agent, tokenizer=tokenizer, gconfig=config.gconfig, mode="online",
                                           proxy_url=switches["proxy"], admin_api_key=admin, turn_discount=0.9,
                                           export_style="individual"))


if __name__ == "__main__":
    main(sys.argv[1:])
