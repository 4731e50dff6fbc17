"""GSM8K builders (areal/dataset/gsm8k.py): RL prompts with the gold answer, and SFT samples."""
from .loaders import load_records, tokenize_prompt_answer

SUFFIX = "\nPlease put your final answer within \\boxed{}."


def rl(path, split="train", tokenizer=None, max_length=None, **kw):
    out = []
    for r in load_records(path, split):
        item = dict(messages=[{"role": "user", "content": r["question"] + SUFFIX}], answer=r["answer"])
        if tokenizer is not None and max_length is not None:
            if len(tokenizer.encode(r["question"])) > max_length:
                continue
        out.append(item)
    return out


def sft(path, split="train", tokenizer=None, max_length=None, **kw):
    assert tokenizer is not None, "SFT dataset needs a tokenizer"
    out = []
    for r in load_records(path, split):
        s = tokenize_prompt_answer(tokenizer, r["question"], r["answer"], max_length)
        if s is not None:
            out.append(s)
    return out


BUILDERS = {("gsm8k", "rl"): rl, ("gsm8k", "sft"): sft}
