"""Small generic helpers (reference ``mindformers/tools/generic.py``): experimental-mode detection for
``from_pretrained`` paths, a context-manager stack, and a ``cached_property``-style helper for config objects."""
from __future__ import annotations

import os
from contextlib import ExitStack, contextmanager
from typing import Iterable


def is_experimental_mode(path: str) -> bool:
    """The reference has two loading conventions: *origin* (a supported model name, or a directory holding a YAML +
    ``.ckpt``) and *experimental* (an HF-like directory with ``config.json``, or a ``repo/name`` id). True for the
    second. A directory with a YAML and no ``config.json`` is origin mode; so is a bare model name."""
    if os.path.isdir(path):
        names = os.listdir(path)
        yaml_here = any(n.endswith((".yaml", ".yml")) for n in names)
        ckpt_here = any(n.endswith(".ckpt") for n in names)
        if "config.json" in names:
            return True
        return not (yaml_here or ckpt_here)
    if path.count("/") == 1 and not path.startswith("mindspore"):
        return True
    return False


@contextmanager
def context_managers(managers: Iterable):
    """Enter several context managers as one."""
    with ExitStack() as stack:
        for m in managers:
            stack.enter_context(m)
        yield


def add_model_info_to_auto_map(auto_map: dict, repo_id: str) -> dict:
    """Prefix every class reference of an ``auto_map`` with ``repo_id--`` (how the hub marks remote code)."""
    out = {}
    for key, value in auto_map.items():
        if isinstance(value, (list, tuple)):
            out[key] = [f"{repo_id}--{v}" if v is not None and "--" not in v else v for v in value]
        elif value is not None and "--" not in value:
            out[key] = f"{repo_id}--{value}"
        else:
            out[key] = value
    return out


class cached_property(property):        # noqa: N801 (name kept for parity with functools / the reference)
    """Property whose value is computed once per instance and kept in ``__<name>``."""

    def __get__(self, obj, objtype=None):
        if obj is None:
            return self
        attr = "__cached_" + self.fget.__name__
        if not hasattr(obj, attr):
            setattr(obj, attr, self.fget(obj))
        return getattr(obj, attr)
