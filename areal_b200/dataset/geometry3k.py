"""Vision-language RL prompts of the geometry3k and ViRL39K layouts: image(s) + question + gold answer
(areal/dataset/geometry3k.py, areal/dataset/virl39k.py). The two corpora use the same record fields, so one
builder serves both registry keys."""
from .loaders import load_records


def rl(path, split="train", tokenizer=None, max_length=None, processor=None, **kw):
    out = []
    for r in load_records(path, split):
        q = r.get("problem") or r.get("question") or r.get("prompt")
        images = r.get("images") or ([r["image"]] if r.get("image") is not None else [])
        content = [{"type": "image", "image": im} for im in images] + [{"type": "text", "text": q}]
        out.append(dict(messages=[{"role": "user", "content": content}], images=images,
                        answer=r.get("answer") or r.get("solution")))
    return out


BUILDERS = {("geometry3k", "rl"): rl, ("virl39k", "rl"): rl}
