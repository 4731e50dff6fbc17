"""JSON-safe envelopes for values that cross the RPC boundary: tensors, numpy arrays,
dataclasses, enums, bytes, tuples/sets, PIL images (as PNG), tokenizers / processors (by the path they
were loaded from), mapping types such as a processor's ``BatchFeature``, and nested containers
(role of areal/infra/rpc/serialization.py in the reference)."""

from __future__ import annotations

import base64
import collections.abc
import dataclasses
import enum
import importlib
import io
from typing import Any

import numpy as np
import torch

_T = "__type__"


def _np_to_b64(a: np.ndarray) -> str:
    buf = io.BytesIO()
    np.save(buf, a, allow_pickle=False)
    return base64.b64encode(buf.getvalue()).decode("ascii")


def _np_from_b64(s: str) -> np.ndarray:
    return np.load(io.BytesIO(base64.b64decode(s)), allow_pickle=False)


def serialize_value(v: Any) -> Any:
    if isinstance(v, float) and (v != v or v in (float("inf"), float("-inf"))):
        return {_T: "float", "value": repr(v)}  # JSON has no inf / nan
    if v is None or isinstance(v, (bool, int, float, str)):
        return v
    if torch.is_tensor(v):
        t = v.detach().cpu()
        if t.dtype == torch.bfloat16:
            return {_T: "tensor", "dtype": "bfloat16", "data": _np_to_b64(t.view(torch.int16).numpy())}
        return {_T: "tensor", "dtype": str(t.dtype).replace("torch.", ""), "data": _np_to_b64(t.numpy())}
    if isinstance(v, np.ndarray):
        return {_T: "ndarray", "data": _np_to_b64(v)}
    if isinstance(v, np.generic):
        return v.item()
    if isinstance(v, bytes):
        return {_T: "bytes", "data": base64.b64encode(v).decode("ascii")}
    if isinstance(v, enum.Enum):
        return {_T: "enum", "cls": f"{type(v).__module__}.{type(v).__qualname__}", "value": v.value}
    if dataclasses.is_dataclass(v) and not isinstance(v, type):
        return {_T: "dataclass", "cls": f"{type(v).__module__}.{type(v).__qualname__}",
                "fields": {f.name: serialize_value(getattr(v, f.name)) for f in dataclasses.fields(v) if f.init}}
    if isinstance(v, dict):
        if all(isinstance(k, str) for k in v) and _T not in v:
            return {k: serialize_value(x) for k, x in v.items()}
        return {_T: "dict", "items": [[serialize_value(k), serialize_value(x)] for k, x in v.items()]}
    if isinstance(v, tuple):
        return {_T: "tuple", "items": [serialize_value(x) for x in v]}
    if isinstance(v, (set, frozenset)):
        return {_T: "set", "items": [serialize_value(x) for x in v]}
    if isinstance(v, list):
        return [serialize_value(x) for x in v]
    if hasattr(v, "__rtensor__"):
        return v.__rtensor__()
    if type(v).__module__.startswith("PIL.") and hasattr(v, "save"):
        buf = io.BytesIO()
        v.save(buf, format="PNG")
        return {_T: "pil", "data": base64.b64encode(buf.getvalue()).decode("ascii")}
    if hasattr(v, "name_or_path") and (hasattr(v, "apply_chat_template") or hasattr(v, "encode")):
        # tokenizers and processors are re-loaded on the other side from where they came from
        kind = "processor" if hasattr(v, "image_processor") else "tokenizer"
        path = v.name_or_path or getattr(getattr(v, "tokenizer", None), "name_or_path", "")
        if not path:
            raise TypeError(f"cannot serialize a {kind} without name_or_path")
        return {_T: kind, "path": path}
    if isinstance(v, collections.abc.Mapping):
        return serialize_value(dict(v))
    raise TypeError(f"cannot serialize value of type {type(v).__name__}")


def _import(path: str):
    mod, _, name = path.rpartition(".")
    obj = importlib.import_module(mod)
    for part in name.split("."):
        obj = getattr(obj, part)
    return obj


def deserialize_value(v: Any) -> Any:
    if isinstance(v, list):
        return [deserialize_value(x) for x in v]
    if not isinstance(v, dict):
        return v
    t = v.get(_T)
    if t is None:
        return {k: deserialize_value(x) for k, x in v.items()}
    if t == "tensor":
        a = _np_from_b64(v["data"])
        if v["dtype"] == "bfloat16":
            return torch.from_numpy(a.copy()).view(torch.bfloat16)
        return torch.from_numpy(a.copy())
    if t == "ndarray":
        return _np_from_b64(v["data"])
    if t == "float":
        return float(v["value"])
    if t == "bytes":
        return base64.b64decode(v["data"])
    if t == "enum":
        return _import(v["cls"])(v["value"])
    if t == "dataclass":
        cls = _import(v["cls"])
        return cls(**{k: deserialize_value(x) for k, x in v["fields"].items()})
    if t == "dict":
        return {deserialize_value(k): deserialize_value(x) for k, x in v["items"]}
    if t == "tuple":
        return tuple(deserialize_value(x) for x in v["items"])
    if t == "set":
        return set(deserialize_value(x) for x in v["items"])
    if t == "pil":
        from PIL import Image

        img = Image.open(io.BytesIO(base64.b64decode(v["data"])))
        img.load()
        return img
    if t == "tokenizer":
        from transformers import AutoTokenizer

        return AutoTokenizer.from_pretrained(v["path"])
    if t == "processor":
        from transformers import AutoProcessor

        return AutoProcessor.from_pretrained(v["path"])
    if t == "rtensor":
        from .rtensor import RTensor

        return RTensor.from_dict(v)
    raise TypeError(f"unknown envelope type {t!r}")
