"""Probing optional packages and comparing their versions."""

from __future__ import annotations

import importlib.metadata
import importlib.util
import re


def is_available(package: str) -> bool:
    try:
        return importlib.util.find_spec(package) is not None
    except (ImportError, ValueError):
        return False


def get_version(package: str) -> str | None:
    try:
        return importlib.metadata.version(package)
    except importlib.metadata.PackageNotFoundError:
        return None


def _key(v: str) -> tuple:
    """Release numbers of a version string, with pre-releases ordered before the release (``1.2.0rc1 < 1.2.0``);
    local parts (``+cu128``) are ignored."""
    v = v.split("+", 1)[0]
    m = re.match(r"^\s*v?(\d+(?:\.\d+)*)(?:[.-]?(a|b|rc|dev|post)\.?(\d*))?", v)
    if not m:
        raise ValueError(f"cannot parse version {v!r}")
    nums = tuple(int(x) for x in m.group(1).split("."))
    nums += (0,) * (4 - len(nums))
    stage = {"dev": -4, "a": -3, "b": -2, "rc": -1, None: 0, "post": 1}[m.group(2)]
    return nums + (stage, int(m.group(3) or 0))


def compare_versions(a: str, b: str) -> int:
    """-1, 0 or 1 as ``a`` is older than, equal to or newer than ``b``."""
    ka, kb = _key(a), _key(b)
    return (ka > kb) - (ka < kb)


def _installed(package: str) -> str:
    v = get_version(package)
    if v is None:
        raise importlib.metadata.PackageNotFoundError(package)
    return v


def is_version_greater_or_equal(package: str, version: str) -> bool:
    return compare_versions(_installed(package), version) >= 0


def is_version_less(package: str, version: str) -> bool:
    return compare_versions(_installed(package), version) < 0


def is_version_equal(package: str, version: str) -> bool:
    return compare_versions(_installed(package), version) == 0
