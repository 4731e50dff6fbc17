"""Rule-based reward functions. Signature used by the workflows:
``reward_fn(prompt, completion, prompt_ids, completion_ids, **dataset_fields) -> float``."""

from .math_parser import extract_answer, math_equal  # noqa: F401
from .gsm8k import gsm8k_reward_fn  # noqa: F401
from .geometry3k import geometry3k_reward_fn  # noqa: F401
from .clevr_count_70k import clevr_count_70k_reward_fn  # noqa: F401


def get_custom_reward_fn(path: str, **kwargs):
    """Dataset path/name → reward function (areal/reward/__init__.py)."""
    p = path.lower()
    if "gsm8k" in p:
        return gsm8k_reward_fn
    if "geometry3k" in p:
        return geometry3k_reward_fn
    if "clevr_count_70k" in p:
        return clevr_count_70k_reward_fn
    raise ValueError(f"no reward function registered for dataset {path!r}")
