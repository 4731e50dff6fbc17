"""ToRL math prompts for tool-integrated reasoning (areal/dataset/torl_data.py)."""
from .loaders import load_records


def rl(path, split="train", tokenizer=None, max_length=None, **kw):
    out = []
    for r in load_records(path, split):
        prompt = r.get("prompt")
        messages = prompt if isinstance(prompt, list) else [{"role": "user", "content": r.get("question") or prompt}]
        answer = r.get("answer")
        if answer is None and isinstance(r.get("reward_model"), dict):
            answer = r["reward_model"].get("ground_truth")
        out.append(dict(messages=messages, answer=answer))
    return out


BUILDERS = {("torl", "rl"): rl}
