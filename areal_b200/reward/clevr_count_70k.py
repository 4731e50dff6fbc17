"""CLEVR counting: integer answer match (areal/reward/clevr_count_70k.py)."""
import re


def clevr_count_70k_reward_fn(prompt, completions, prompt_ids, completion_ids, answer=None, **kwargs) -> float:
    m = re.findall(r"\[(\d+)\]|(?<![\d.])(\d+)(?![\d.])", completions or "")
    nums = [a or b for a, b in m]
    try:
        return float(bool(nums) and int(nums[-1]) == int(str(answer).strip()))
    except ValueError:
        return 0.0
