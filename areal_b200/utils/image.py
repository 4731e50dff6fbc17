"""Image helpers of the vision-language workflows: PIL images to base64 payloads, batches padded to one size."""

from __future__ import annotations

import base64
from io import BytesIO
from typing import Sequence


def image2base64(images) -> list[str]:
    """PNG-encodes one PIL image or a list of them; returns base64 strings (the payload of ``image_url`` parts and
    of the HTTP rollout servers)."""
    from PIL.Image import Image as ImageObject

    if isinstance(images, ImageObject):
        images = [images]
    out = []
    for img in images:
        with BytesIO() as buf:
            img.save(buf, format="PNG")
            out.append(base64.b64encode(buf.getvalue()).decode("utf-8"))
    return out


def base642image(data: str):
    """Inverse of :func:`image2base64` for one string (a ``data:...;base64,`` prefix is accepted)."""
    from PIL import Image

    if data.startswith("data:"):
        data = data.split(",", 1)[1]
    return Image.open(BytesIO(base64.b64decode(data))).convert("RGB")


def pad_images_batch_to_max_size(images: Sequence, fill=(0, 0, 0)) -> list:
    """Every image centred on a canvas of the batch's largest width and height."""
    from PIL import Image

    w, h = max(i.size[0] for i in images), max(i.size[1] for i in images)
    out = []
    for img in images:
        canvas = Image.new("RGB", (w, h), fill)
        canvas.paste(img, ((w - img.size[0]) // 2, (h - img.size[1]) // 2))
        out.append(canvas)
    return out
