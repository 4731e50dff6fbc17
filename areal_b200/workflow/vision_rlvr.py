"""Single-turn RLVR for vision-language prompts.

The processor turns ``messages`` + ``images`` into token ids and pixel tensors; the request
carries the images (base64 PNG) to the inference engine and the trajectory keeps the processor's
``multi_modal_input`` next to the usual token-level fields so a vision-language train engine can
recompute logprobs. Behaviour of areal/workflow/vision_rlvr.py in the reference. The in-process
rollout engine serves Qwen2.5-VL and reads the processor's tensors straight from the request's
metadata; an engine that does not accept images (a text-only model) rejects the request with a
clear error rather than silently dropping them.
"""

from __future__ import annotations

import base64
import io
import uuid
from typing import Any

import torch

from ..api.io_struct import ModelRequest
from ..utils import stats_tracker
from .rlvr import RLVRWorkflow


def image_to_base64(img) -> str:
    """PIL image (or raw PNG bytes) → base64 PNG string."""
    if isinstance(img, (bytes, bytearray)):
        return base64.b64encode(bytes(img)).decode()
    buf = io.BytesIO()
    img.save(buf, format="PNG")
    return base64.b64encode(buf.getvalue()).decode()


def load_image(obj, decode_bytes: bool = True):
    """What a dataset row holds for an image → PIL image: a ``{"bytes": ..., "path": ...}`` record (parquet /
    ``datasets`` image feature), encoded bytes, or a file path; PIL images pass through. With
    ``decode_bytes=False`` raw bytes are left alone (a processor that takes them as they are)."""
    if isinstance(obj, dict):
        obj = obj.get("bytes") or obj.get("path")
    if isinstance(obj, (bytes, bytearray)) and decode_bytes:
        from PIL import Image

        try:
            return Image.open(io.BytesIO(bytes(obj))).convert("RGB")
        except Exception:
            return obj  # not an encoded image: hand it to the processor unchanged
    if isinstance(obj, str):
        from PIL import Image

        return Image.open(obj).convert("RGB")
    return obj


class VisionRLVRWorkflow(RLVRWorkflow):
    def __init__(self, reward_fn, gconfig, tokenizer, processor, enable_thinking: bool = False, **kw):
        super().__init__(reward_fn, gconfig, tokenizer=tokenizer, enable_thinking=enable_thinking, **kw)
        self.processor = processor

    async def arun_episode(self, engine, data: dict[str, Any]):
        images = [load_image(im) for im in (data.get("images") or [])]
        text = self.processor.apply_chat_template(data["messages"], tokenize=False, add_generation_prompt=True) \
            if "messages" in data else data["prompt"]
        proc = self.processor(images=images or None, text=text, padding=False, return_tensors="pt")
        input_ids = proc["input_ids"][0].tolist()
        mm = {k: v for k, v in proc.items() if k not in ("input_ids", "attention_mask")}
        # an in-process engine reads the processor's tensors from the metadata; a remote server gets the encoded
        # images and runs its own processor
        req = ModelRequest(rid=uuid.uuid4().hex, input_ids=input_ids, gconfig=self.gconfig, tokenizer=self.tokenizer,
                           image_data=[image_to_base64(i) for i in images] or None, processor=self.processor,
                           metadata={"multi_modal_input": [mm]} if images else {})
        if images and not getattr(engine, "supports_images", False):
            raise NotImplementedError(f"{type(engine).__name__} is a text-only engine: it cannot serve image prompts")
        resp = await engine.agenerate(req)
        completion = self.tokenizer.decode(resp.output_tokens)
        reward = await self._reward(self.tokenizer.decode(input_ids), completion, resp.input_tokens, resp.output_tokens,
                                    {k: v for k, v in data.items() if k != "images"})
        stats_tracker.get("rollout").scalar(reward=reward, gen_len=float(resp.output_len))
        seq = resp.input_tokens + resp.output_tokens
        n_in, n_out = resp.input_len, resp.output_len
        return dict(
            input_ids=torch.tensor(seq, dtype=torch.int32).unsqueeze(0),
            attention_mask=torch.ones(1, len(seq), dtype=torch.bool),
            loss_mask=torch.tensor([0] * n_in + [1] * n_out, dtype=torch.int32).unsqueeze(0),
            logprobs=torch.tensor([0.0] * n_in + resp.output_logprobs, dtype=torch.float32).unsqueeze(0),
            versions=torch.tensor([-1] * n_in + resp.output_versions, dtype=torch.int32).unsqueeze(0),
            rewards=torch.tensor([float(reward)], dtype=torch.float32),
            multi_modal_input=[mm],
        )
