"""Declarative module specs (``ModuleSpec`` + ``build_module``), as in Megatron-Core.

Same role as the reference's ``parallel_core/utils/spec_utils.py`` (:9-28, :58-106): a layer is
described by the class to instantiate, fixed keyword arguments, and the specs of its sub-modules,
so that model variants differ in specs rather than in code.
"""
from __future__ import annotations

import importlib
from dataclasses import dataclass, field
from typing import Any, Tuple, Union


@dataclass
class ModuleSpec:
    """``module`` (a class, a ``(module path, name)`` pair or a callable) + fixed ``params`` + the specs of its
    ``submodules``."""

    module: Union[type, Tuple[str, str], Any]
    params: dict = field(default_factory=dict)
    submodules: Any = None


def import_module(path: Tuple[str, str]):
    mod, name = path
    return getattr(importlib.import_module(mod), name)


def build_module(spec_or_module, *args, **kwargs):
    """Instantiate a ``ModuleSpec`` (or a bare class); functions are returned as they are."""
    if spec_or_module is None:
        return None
    if isinstance(spec_or_module, ModuleSpec):
        target, params, subs = spec_or_module.module, dict(spec_or_module.params), spec_or_module.submodules
    else:
        target, params, subs = spec_or_module, {}, None
    if isinstance(target, tuple):
        target = import_module(target)
    if not isinstance(target, type):
        if callable(target) and not args and not kwargs and not params:
            return target
    if subs is not None:
        kwargs = dict(kwargs, submodules=subs)
    params.update(kwargs)
    try:
        return target(*args, **params)
    except Exception as e:  # add the failing module's name to the message
        raise type(e)(f"{getattr(target, '__name__', target)}: {e}").with_traceback(e.__traceback__) from None
