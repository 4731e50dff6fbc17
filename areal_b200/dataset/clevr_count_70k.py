"""clevr_count_70k: image(s) + counting question + gold answer (areal/dataset/clevr_count_70k.py).

``rl``: prompts for the vision RLVR workflow. ``sft``: token ids with the image placeholders expanded by the
processor, a loss mask over the answer tokens and the processor's pixel tensors as ``multi_modal_input``."""
import math

from .loaders import load_records

QWEN_IMAGE_TOKEN = "<|vision_start|><|image_pad|><|vision_end|>"


def _images(r):
    return r.get("images") or ([r["image"]] if r.get("image") is not None else [])


def shrink_image(img, max_pixels: int | None):
    """Down-scales a PIL image to at most ``max_pixels`` (aspect kept); other objects pass through."""
    if max_pixels is None or not hasattr(img, "resize") or img.width * img.height <= max_pixels:
        return img
    f = math.sqrt(max_pixels / (img.width * img.height))
    return img.resize((max(int(img.width * f), 1), max(int(img.height * f), 1)))


def rl(path, split="train", tokenizer=None, max_length=None, processor=None, **kw):
    out = []
    for r in load_records(path, split):
        q = r.get("problem") or r.get("question") or r.get("prompt")
        images = _images(r)
        content = [{"type": "image", "image": im} for im in images] + [{"type": "text", "text": q}]
        out.append(dict(messages=[{"role": "user", "content": content}], images=images,
                        answer=r.get("answer") or r.get("solution")))
    return out


def sft(path, split="train", tokenizer=None, max_length=None, processor=None, max_pixels: int | None = 336 * 336,
        image_token: str | None = None, **kw):
    if processor is None:
        raise ValueError("the vision-language SFT dataset needs the model's processor")
    tok = tokenizer or processor.tokenizer
    image_token = image_token or getattr(processor, "image_token_with_markers", None) or QWEN_IMAGE_TOKEN
    out = []
    for r in load_records(path, split):
        images = [shrink_image(im, max_pixels) for im in _images(r)]
        problem = (r.get("problem") or r.get("question") or "").replace("<image>", image_token)
        answer = str(r.get("answer") or r.get("solution") or "")
        proc = processor(text=[problem + answer + (tok.eos_token or "")], images=images or None, padding=False,
                         return_tensors="pt")
        ids = proc["input_ids"][0].tolist()
        if max_length is not None and len(ids) > max_length:
            continue
        n_ans = len(tok.encode(answer, add_special_tokens=False)) + (1 if tok.eos_token else 0)
        item = dict(input_ids=ids, loss_mask=[0] * (len(ids) - n_ans) + [1] * n_ans)
        if images:
            item["multi_modal_input"] = [{k: v for k, v in proc.items() if k not in ("input_ids", "attention_mask")}]
        out.append(item)
    return out


BUILDERS = {("clevr_count_70k", "rl"): rl, ("clevr_count_70k", "sft"): sft}
