"""Re-exporting selected methods of one object on another (areal/utils/wrapper.py): an engine marks the methods
that a controller or an RPC proxy should expose with ``@wrapable()``, and ``wrap(target, source, transform)``
installs them on ``target``, optionally routed through ``transform`` (which receives the method's name and the
original bound method as keyword arguments and removes them with ``wrap_remove_meta`` before calling on)."""

from __future__ import annotations

import inspect
from functools import partial
from typing import Any, Callable

_NAME, _ORIG = "wrap_method_name", "wrap_original_method"


def wrapable(name: str | None = None):
    def mark(fn):
        fn.__wrap_meta__ = {"name": name or fn.__name__}
        return fn

    return mark


def wrap(target: object, source: object, transform: Callable[..., Any] | None = None) -> list[str]:
    """Installs every ``@wrapable`` method of ``source`` on ``target``; returns the installed names."""
    names = []
    for _, member in inspect.getmembers(source, callable):
        meta = getattr(member, "__wrap_meta__", None)
        if meta is None:
            continue
        name = meta["name"]
        setattr(target, name, member if transform is None else partial(transform, **{_NAME: name, _ORIG: member}))
        names.append(name)
    return names


def wrap_get_method_name(kwargs: dict) -> str:
    return kwargs[_NAME]


def wrap_get_method(kwargs: dict) -> Callable:
    return kwargs[_ORIG]


def wrap_remove_meta(kwargs: dict) -> dict:
    kwargs.pop(_NAME, None)
    kwargs.pop(_ORIG, None)
    return kwargs
