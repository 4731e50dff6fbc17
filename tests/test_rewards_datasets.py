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


def test_countdown_reward_and_dataset(tmp_path):
    from fractions import Fraction

    from areal_b200.dataset import get_custom_dataset
    from areal_b200.dataset.countdown import generate
    from areal_b200.reward.countdown import countdown_reward_fn, countdown_score, evaluate, extract_answer

    assert evaluate("(7 - (5 - 3)) * 8") == 40 and evaluate("8 / 3 * 3") == 8 and evaluate("-3 + 5") == 2
    assert evaluate("2 +") is None and evaluate("4 / (2 - 2)") is None and evaluate("2 ** 3") is None
    assert evaluate("__import__('os')") is None and evaluate("") is None and evaluate("(1 + 2") is None
    assert evaluate("7 / 2") == Fraction(7, 2)
    assert extract_answer("<think>x</think> <answer> (3 + 5) * 3 = 24 </answer>") == "(3 + 5) * 3"
    assert countdown_score("no tags", 24, [3, 5, 3]) == 0.0
    assert countdown_score("<answer>(3 + 5) * 3</answer>", 24, [3, 5, 3]) == 1.0
    assert countdown_score("<answer>(3 + 5) * 4</answer>", 24, [3, 5, 3]) == 0.1      # a number that was not given
    assert countdown_score("<answer>3 + 5 + 3</answer>", 24, [3, 5, 3]) == 0.1        # wrong value
    assert countdown_score("<answer>3 + 5</answer>", 8, [3, 5, 3]) == 0.1             # one number unused
    assert countdown_score("<answer>1</answer> <answer>5 * 5 - 1</answer>", 24, [5, 5, 1]) == 1.0  # the last block counts
    d = tmp_path / "countdown"
    generate(str(d / "train.jsonl"), 50, seed=3)
    items = get_custom_dataset(path=str(d), type="rl", split="train")
    assert len(items) == 50
    import json

    for it, line in zip(items, open(d / "train.jsonl")):
        rec = json.loads(line)
        assert str(it["target"]) in it["messages"][0]["content"] and len(it["numbers"]) == 4
        # the recorded solution solves its own puzzle through the reward function
        assert countdown_reward_fn("", f"<answer>{rec['solution']}</answer>", [], [], **it) == 1.0
