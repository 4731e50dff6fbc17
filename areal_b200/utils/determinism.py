"""Deterministic-mode switches (``megatron.use_deterministic_algorithms``).

Bit-stable runs need every reduction to happen in one fixed order. With the switch on:

* ``torch.use_deterministic_algorithms(True, warn_only=True)`` and the cuBLAS workspace setting cover
  the PyTorch operators that remain on the path;
* NCCL reductions use the ring algorithm (a fixed summation order for a fixed topology);
* the two kernels of this library that sum through floating-point atomics step aside: the embedding
  gradient takes the sorted PyTorch scatter (``ops/fused.py``) and the attention backward, whose dQ tiles
  are accumulated with ``red.global.add`` in arrival order, is recomputed through the PyTorch formulation
  (``ops/attention.py``; quadratic memory per sequence, meant for debugging runs, not for long contexts).

Everything else in the library (GEMMs with fp32 accumulation in TMEM, fused LM head, norms, optimizer,
peer reduce-scatter with a fixed peer order) is deterministic as it stands.
Reference: areal/engine/megatron_utils/deterministic.py:12-44.
"""

from __future__ import annotations

import os

import torch

from . import logging

logger = logging.getLogger("Determinism")

_enabled = False


def deterministic_mode() -> bool:
    return _enabled


def set_deterministic_algorithms(enabled: bool = True) -> None:
    global _enabled
    _enabled = bool(enabled)
    if not enabled:
        torch.use_deterministic_algorithms(False)
        return
    if os.environ.get("NCCL_ALGO") not in ("Tree", "Ring", "CollnetDirect", "CollnetChain", "^NVLS"):
        logger.info("deterministic mode: NCCL_ALGO set to 'Ring'")
        os.environ["NCCL_ALGO"] = "Ring"
    if os.environ.get("CUBLAS_WORKSPACE_CONFIG") not in (":4096:8", ":16:8"):
        os.environ["CUBLAS_WORKSPACE_CONFIG"] = ":4096:8"
    torch.use_deterministic_algorithms(True, warn_only=True)
