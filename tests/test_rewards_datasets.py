"""Reward parsers and local-file dataset builders."""
import json

import pytest

from areal_b200.dataset import get_custom_dataset
from areal_b200.reward import extract_answer, get_custom_reward_fn, gsm8k_reward_fn, math_equal
from areal_b200.reward.clevr_count_70k import clevr_count_70k_reward_fn
from areal_b200.reward.geometry3k import geometry3k_reward_fn


@pytest.mark.parametrize("text,ans", [
    ("so the total is \\boxed{42}.", "42"), ("… #### 1,234", "1,234"), ("The answer is 3/4.", "3/4"),
    ("first 3 then 10 and finally 7", "7"), ("\\boxed{\\frac{1}{2}}", "\\frac{1}{2}"), ("no number", None)])
def test_extract_answer(text, ans):
    assert extract_answer(text) == ans


@pytest.mark.parametrize("a,b,eq", [("42", "42.0", True), ("1,234", "1234", True), ("\\frac{1}{2}", "0.5", True),
                                    ("50%", "0.5", True), ("3/4", "0.75", True), ("7", "8", False), (None, "1", False),
                                    ("$18$", "18", True), ("x+1", "X+1", True)])
def test_math_equal(a, b, eq):
    assert math_equal(a, b) is eq


def test_reward_functions():
    assert gsm8k_reward_fn("q", "we get \\boxed{18}", [], [], answer="blah #### 18") == 1.0
    assert gsm8k_reward_fn("q", "we get 17", [], [], answer="#### 18") == 0.0
    assert geometry3k_reward_fn("q", "thus [12.5]", [], [], answer="12.5") == 1.0
    assert clevr_count_70k_reward_fn("q", "there are [3] objects", [], [], answer="3") == 1.0
    assert clevr_count_70k_reward_fn("q", "none", [], [], answer="3") == 0.0
    assert get_custom_reward_fn("openai/gsm8k") is gsm8k_reward_fn
    with pytest.raises(ValueError):
        get_custom_reward_fn("unknown")


class _Tok:
    eos_token_id = 2

    def encode(self, s, add_special_tokens=True):
        return [3 + (ord(c) % 50) for c in s]


def test_dataset_builders(tmp_path):
    d = tmp_path / "gsm8k"
    d.mkdir()
    with open(d / "train.jsonl", "w") as f:
        for i in range(3):
            f.write(json.dumps({"question": f"what is {i}+1?", "answer": f"it is #### {i + 1}"}) + "\n")
    rl = get_custom_dataset(str(d), type="rl")
    assert len(rl) == 3 and rl[0]["messages"][0]["role"] == "user" and rl[2]["answer"].endswith("3")
    sft = get_custom_dataset(str(d), type="sft", tokenizer=_Tok())
    assert len(sft[0]["input_ids"]) == len(sft[0]["loss_mask"]) and sft[0]["loss_mask"][-1] == 1 and sft[0]["loss_mask"][0] == 0
    h = tmp_path / "hh-rlhf"
    h.mkdir()
    with open(h / "train.jsonl", "w") as f:
        f.write(json.dumps({"chosen": "Human: hi Assistant: hello there", "rejected": "Human: hi Assistant: go away"}) + "\n")
    pairs = get_custom_dataset(str(h), type="dpo", tokenizer=_Tok())
    assert pairs[0]["chosen_ids"][:5] == pairs[0]["rejected_ids"][:5] and sum(pairs[0]["chosen_loss_mask"]) > 0
    with pytest.raises(ValueError):
        get_custom_dataset(str(d), type="dpo")
