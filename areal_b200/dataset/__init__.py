"""Dataset registry. ``get_custom_dataset(path=..., type=..., split=..., tokenizer=...)`` returns a
list-like of dict items in the shape the trainers expect (areal/dataset/__init__.py):

* ``type="rl"``  – ``{"messages": [...], "answer": ...}`` (prompt only; the workflow generates)
* ``type="sft"`` – ``{"input_ids", "loss_mask"}``
* ``type="rw"`` / ``"dpo"`` – ``{"chosen_ids", "rejected_ids", "chosen_loss_mask", "rejected_loss_mask"}``

Data is read from local files (``.jsonl``, ``.json``, ``.parquet`` or a ``datasets`` directory saved
with ``save_to_disk``); nothing is downloaded.
"""

from __future__ import annotations

import json
import os
from typing import Any, Callable

from .loaders import load_records
from . import gsm8k, hhrlhf, geometry3k, clevr_count_70k, torl_data, countdown, agent_tasks  # noqa: F401

_REGISTRY: dict[tuple[str, str], Callable] = {}


def register(name: str, type_: str):
    def deco(fn):
        _REGISTRY[(name, type_)] = fn
        return fn

    return deco


for _mod in (gsm8k, hhrlhf, geometry3k, clevr_count_70k, torl_data, countdown, agent_tasks):
    for (_n, _t), _f in getattr(_mod, "BUILDERS", {}).items():
        _REGISTRY[(_n, _t)] = _f


def get_custom_dataset(path: str, type: str = "rl", split: str = "train", tokenizer=None, max_length: int | None = None,
                       processor=None, **kwargs) -> list[dict[str, Any]]:
    key = next((n for (n, t) in _REGISTRY if n in path.lower() and t == type), None)
    if key is None:
        raise ValueError(f"no dataset builder for path={path!r} type={type!r}; known: {sorted(_REGISTRY)}")
    return _REGISTRY[(key, type)](path=path, split=split, tokenizer=tokenizer, max_length=max_length,
                                  processor=processor, **kwargs)
