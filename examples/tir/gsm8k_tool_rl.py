"""Tool-integrated reasoning on GSM8K: the policy must call calculator tools (function calling over the
chat-completions protocol) and is rewarded for the final answer; tool-calling turns share the reward
through the turn discount.

    python -m areal_b200.infra.launcher.local examples/tir/gsm8k_tool_rl.py \
        --config examples/math/gsm8k_grpo.yaml experiment_name=gsm8k-tir
"""
import importlib.util
import os
import sys


def main(argv):
    here = os.path.dirname(os.path.abspath(__file__))
    spec = importlib.util.spec_from_file_location(
        "gsm8k_agent_rl", os.path.join(here, "..", "openai_agent", "gsm8k_agent_rl.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    mod.main(argv, default_agent="tool")


if __name__ == "__main__":
    main(sys.argv[1:])
