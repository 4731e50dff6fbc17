"""Anthropic HH-RLHF preference pairs for reward-model and DPO training (areal/dataset/hhrlhf.py)."""
from .loaders import load_records


def _split_prompt(chosen: str, rejected: str):
    i = 0
    n = min(len(chosen), len(rejected))
    while i < n and chosen[i] == rejected[i]:
        i += 1
    cut = chosen.rfind("Assistant:", 0, i + 1)
    cut = cut + len("Assistant:") if cut >= 0 else i
    return chosen[:cut], chosen[cut:], rejected[cut:]


def pairs(path, split="train", tokenizer=None, max_length=None, **kw):
    assert tokenizer is not None, "preference datasets need a tokenizer"
    eos = [tokenizer.eos_token_id] if getattr(tokenizer, "eos_token_id", None) is not None else []
    out = []
    for r in load_records(path, split):
        prompt, c, rj = _split_prompt(r["chosen"], r["rejected"])
        p = tokenizer.encode(prompt)
        ci = tokenizer.encode(c, add_special_tokens=False) + eos
        ri = tokenizer.encode(rj, add_special_tokens=False) + eos
        if max_length is not None and max(len(p) + len(ci), len(p) + len(ri)) > max_length:
            continue
        out.append(dict(chosen_ids=p + ci, rejected_ids=p + ri,
                        chosen_loss_mask=[0] * len(p) + [1] * len(ci),
                        rejected_loss_mask=[0] * len(p) + [1] * len(ri)))
    return out


BUILDERS = {("hh-rlhf", "rw"): pairs, ("hh-rlhf", "dpo"): pairs, ("hhrlhf", "rw"): pairs, ("hhrlhf", "dpo"): pairs}
