"""Random-generator state in recover checkpoints: one small file per rank (``rng/rank00003.pt``) with the states
of Python's ``random``, NumPy's global generator, torch's CPU generator and, on a GPU, the current device's
generator. A run that resumes with the same number of ranks continues the random streams it stopped in (dropout
masks, sampling noise drawn on the trainer side, shuffles that use the global generators); with another number of
ranks the per-rank streams have no counterpart, so the files are ignored and the run re-seeds from its
configuration.
Reference: the per-rank RNG entries of Megatron's distributed checkpoints, saved through
areal/engine/megatron_utils/checkpointer.py (``get_rng_state``)."""

from __future__ import annotations

import os
import random

import numpy as np
import torch

from . import logging

logger = logging.getLogger("rng_state")


def _file(path: str, rank: int) -> str:
    return os.path.join(path, "rng", f"rank{rank:05d}.pt")


def capture(device: torch.device | None = None) -> dict:
    state = {"python": random.getstate(), "numpy": np.random.get_state(), "torch_cpu": torch.get_rng_state()}
    if device is not None and device.type == "cuda":
        state["torch_cuda"] = torch.cuda.get_rng_state(device)
    return state


def restore(state: dict, device: torch.device | None = None) -> None:
    random.setstate(state["python"])
    np.random.set_state(state["numpy"])
    torch.set_rng_state(state["torch_cpu"])
    if "torch_cuda" in state and device is not None and device.type == "cuda":
        torch.cuda.set_rng_state(state["torch_cuda"], device)


def save_rng_state(path: str, rank: int, world_size: int, device: torch.device | None = None) -> str:
    f = _file(path, rank)
    os.makedirs(os.path.dirname(f), exist_ok=True)
    tmp = f + ".tmp"
    torch.save({"world_size": world_size, "state": capture(device)}, tmp)
    os.replace(tmp, f)
    return f


def load_rng_state(path: str, rank: int, world_size: int, device: torch.device | None = None) -> bool:
    """Restores this rank's generators; False (and nothing touched) when the checkpoint has no entry for it or was
    written by a job of another size."""
    f = _file(path, rank)
    if not os.path.exists(f):
        return False
    blob = torch.load(f, map_location="cpu", weights_only=False)
    if int(blob.get("world_size", -1)) != world_size:
        logger.warning(f"the checkpoint's random-generator states are of a {blob.get('world_size')}-rank job, this "
                       f"one has {world_size} ranks: not restored")
        return False
    restore(blob["state"], device)
    return True
