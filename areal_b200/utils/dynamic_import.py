"""Resolving objects named in configs and RPC payloads (areal/utils/dynamic_import.py).

``"pkg.mod.attr"`` and ``"pkg.mod:attr"`` import a module and take an attribute (dotted attributes allowed after
the colon); ``"/path/to/file.py:attr"`` loads a source file that is not on ``sys.path`` (user scripts that a
scheduler worker has to import by path)."""

from __future__ import annotations

import hashlib
import importlib
import importlib.util
import os
import sys
from typing import Any


def _walk(obj: Any, dotted: str) -> Any:
    for part in dotted.split("."):
        obj = getattr(obj, part)
    return obj


def import_from_string(path: str) -> Any:
    if not isinstance(path, str) or not path:
        raise ValueError(f"expected a dotted path, got {path!r}")
    mod_part, sep, attr = path.partition(":")
    if sep and (mod_part.endswith(".py") or os.sep in mod_part):
        file = os.path.abspath(mod_part)
        name = "_dyn_" + hashlib.sha1(file.encode()).hexdigest()[:12]
        module = sys.modules.get(name)
        if module is None:
            spec = importlib.util.spec_from_file_location(name, file)
            if spec is None or spec.loader is None:
                raise ImportError(f"cannot load {file}")
            module = importlib.util.module_from_spec(spec)
            sys.modules[name] = module
            try:
                spec.loader.exec_module(module)
            except BaseException:
                sys.modules.pop(name, None)
                raise
        return _walk(module, attr)
    if sep:
        return _walk(importlib.import_module(mod_part), attr)
    mod_part, _, attr = path.rpartition(".")
    if not mod_part:
        return importlib.import_module(path)
    try:
        return getattr(importlib.import_module(mod_part), attr)
    except AttributeError:
        # "pkg.mod" given as a whole: the last component is itself a module
        try:
            return importlib.import_module(path)
        except ImportError:
            raise ImportError(f"module {mod_part!r} has no attribute {attr!r}") from None
