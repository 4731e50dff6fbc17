"""Rollout through an inference service: several rollout-engine workers behind one gateway, and a script that uses
them like a local engine.

    # 1. the gateway (with a tokenizer it also serves /v1/chat/completions)
    python -m uvicorn --factory areal_b200.services.inference_service:create_gateway_app --port 9000
    # 2. engine workers (each an RPC server hosting a rollout engine) register themselves:
    #    POST http://gateway:9000/register {"worker_id": "w0", "addr": "host0:8100"}
    # 3. this script
    python examples/inference_service/rollout_via_gateway.py --config examples/math/gsm8k_grpo.yaml \
        gateway=http://gateway:9000 train_dataset.path=/data/gsm8k

`GatewayInferenceEngine` implements the inference-engine interface over the gateway's routes, so workflows,
`rollout_batch` and `prepare_batch` work unchanged; multi-turn workflows can pin a conversation to the engine that
holds its prefix with `start_session` / `finish_session`.
"""
import sys

from areal_b200.api.cli_args import GRPOConfig, load_expr_config
from areal_b200.dataset import get_custom_dataset
from areal_b200.services.inference_service import GatewayInferenceEngine
from areal_b200.utils.hf_io import load_hf_tokenizer
from areal_b200.workflow.rlvr import RLVRWorkflow


def pop_switches(argv):
    mine, rest = {}, []
    for a in argv:
        k, _, v = a.partition("=")
        if k in ("gateway", "token", "n"):
            mine[k] = v
        else:
            rest.append(a)
    return mine, rest


def main(argv):
    switches, argv = pop_switches(list(argv))
    if "gateway" not in switches:
        raise SystemExit("give gateway=<url of the inference gateway>")
    config, _ = load_expr_config(argv, GRPOConfig)
    tokenizer = load_hf_tokenizer(config.tokenizer_path or config.actor.path)
    data = get_custom_dataset(path=config.train_dataset.path, type="rl", split="train", tokenizer=tokenizer)
    engine = GatewayInferenceEngine(config.rollout, switches["gateway"], token=switches.get("token")).initialize()
    try:
        wf = RLVRWorkflow(reward_fn="areal_b200.reward.gsm8k.gsm8k_reward_fn", gconfig=config.gconfig.new(n_samples=1),
                          tokenizer=tokenizer)
        n = int(switches.get("n", 64))
        batch = engine.rollout_batch([data[i] for i in range(min(n, len(data)))], workflow=wf)
        print(f"{batch['rewards'].numel()} samples, mean reward {batch['rewards'].float().mean():.4f}, "
              f"mean length {batch['attention_mask'].sum(-1).float().mean():.1f} tokens")
    finally:
        engine.destroy()


if __name__ == "__main__":
    main(sys.argv[1:])
