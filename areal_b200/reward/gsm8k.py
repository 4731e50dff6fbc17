"""GSM8K: reward 1 when the completion's final answer equals the reference (areal/reward/gsm8k.py)."""
from .math_parser import extract_answer, math_equal


def gsm8k_reward_fn(prompt, completions, prompt_ids, completion_ids, answer=None, **kwargs) -> float:
    ref = extract_answer(str(answer)) if answer is not None and "####" in str(answer) else answer
    return float(math_equal(extract_answer(completions), None if ref is None else str(ref)))
