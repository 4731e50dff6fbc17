"""Geometry3K: answers are given in ``[...]`` brackets or boxed (areal/reward/geometry3k.py)."""
import re

from .math_parser import extract_answer, math_equal


def geometry3k_reward_fn(prompt, completions, prompt_ids, completion_ids, answer=None, **kwargs) -> float:
    m = re.findall(r"\[([^\[\]]+)\]", completions or "")
    pred = m[-1] if m else extract_answer(completions)
    return float(math_equal(pred, None if answer is None else str(answer)))
