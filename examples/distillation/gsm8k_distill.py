"""GRPO on GSM8K with on-policy distillation from a teacher model (`teacher:` block of the config).

    python -m areal_b200.infra.launcher.local examples/distillation/gsm8k_distill.py \
        --config examples/distillation/gsm8k_grpo_distill.yaml actor.path=/models/Qwen3-1.7B teacher.path=/models/Qwen3-8B
"""
import importlib.util
import os
import sys


def main(argv):
    here = os.path.dirname(os.path.abspath(__file__))
    spec = importlib.util.spec_from_file_location("gsm8k_rl", os.path.join(here, "..", "math", "gsm8k_rl.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    mod.main(argv)  # the trainer builds the teacher engine whenever the config has a `teacher` block


if __name__ == "__main__":
    main(sys.argv[1:])
