"""Deterministic seeding: one base seed, a distinct stream per (key) via hashing
(areal/utils/seeding.py)."""

from __future__ import annotations

import hashlib
import random

import numpy as np
import torch

_BASE_SEED: int | None = None
_SEED: int | None = None


def _mix(seed: int, key: str) -> int:
    h = hashlib.sha256(f"{seed}:{key}".encode()).digest()
    return int.from_bytes(h[:4], "little")


def set_random_seed(base_seed: int, key: str = "") -> int:
    global _BASE_SEED, _SEED
    _BASE_SEED = base_seed
    seed = _mix(base_seed, key) if key else base_seed
    _SEED = seed
    random.seed(seed)
    np.random.seed(seed % (2 ** 32))
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)
    return seed


def get_seed() -> int:
    if _SEED is None:
        raise RuntimeError("set_random_seed has not been called")
    return _SEED


def get_shuffle_seed() -> int:
    if _BASE_SEED is None:
        raise RuntimeError("set_random_seed has not been called")
    return _mix(_BASE_SEED, "shuffle")


class Shuffler:
    """A stream of shuffle seeds derived from a key: call ``next_shuffle()`` once per epoch (or per shuffle); two
    shufflers with the same key produce the same stream."""

    def __init__(self, key: str = "default"):
        self.base_key, self.cnt = key, 0

    def next_shuffle(self) -> int:
        seed = _mix(0, f"{self.base_key}_{self.cnt}")
        self.cnt += 1
        return seed

    def state_dict(self) -> dict:
        return {"key": self.base_key, "cnt": self.cnt}

    def load_state_dict(self, s: dict) -> None:
        self.base_key, self.cnt = s["key"], int(s["cnt"])
