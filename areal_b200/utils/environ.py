"""Boolean switches read from the environment."""

from __future__ import annotations

import os

from . import logging

logger = logging.getLogger("environ")
_warned: set[str] = set()


def get_bool_env_var(name: str, default: str = "false") -> bool:
    """``true`` / ``1`` → True, ``false`` / ``0`` → False (case-insensitive); anything else counts as False and is
    reported once per variable."""
    raw = os.getenv(name, default).strip().lower()
    if raw in ("true", "1", "yes", "on"):
        return True
    if raw not in ("false", "0", "no", "off", "") and name not in _warned:
        _warned.add(name)
        logger.warning(f"{name}={raw!r} is not a boolean; treated as false")
    return False


def is_in_ci() -> bool:
    return get_bool_env_var("AREAL_IS_IN_CI")


def is_single_controller() -> bool:
    """True unless the process runs as one rank of an SPMD launch (``RANK`` set by torchrun, or
    ``AREAL_SPMD_MODE=1``)."""
    return not (get_bool_env_var("AREAL_SPMD_MODE") or "RANK" in os.environ)
