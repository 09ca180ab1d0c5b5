"""``import mindformers`` for code written against the reference's package name.

The implementation lives in ``mindformers_b200``; this package makes every name and every sub-module of it importable
under ``mindformers`` (``from mindformers import Trainer, AutoModel``, ``from mindformers.tools.register import
MindFormerConfig``, ``import mindformers.core.context``), so a script of the reference's API surface
(``mindformers/__init__.py:20-245`` there) runs without edits. Sub-modules are aliases, not copies: ``mindformers.x``
and ``mindformers_b200.x`` are the same module object.
"""
from __future__ import annotations

import importlib
import importlib.abc
import importlib.util
import sys

import mindformers_b200 as _impl

__version__ = _impl.__version__
__all__ = list(_impl.__all__)

_PREFIX, _TARGET = __name__ + ".", _impl.__name__ + "."


class _AliasLoader(importlib.abc.Loader):
    def __init__(self, target: str):
        self.target = target

    def create_module(self, spec):
        module = importlib.import_module(self.target)    # the very module object of the implementation
        self._spec = module.__spec__                     # the import system rebinds ``__spec__`` to the alias's
        return module

    def exec_module(self, module):
        module.__spec__ = self._spec


class _AliasFinder(importlib.abc.MetaPathFinder):
    """Resolves ``mindformers.<path>`` to ``mindformers_b200.<path>``."""

    def find_spec(self, fullname, path=None, target=None):
        if not fullname.startswith(_PREFIX):
            return None
        real = _TARGET + fullname[len(_PREFIX):]
        try:
            found = importlib.util.find_spec(real)
        except (ImportError, ValueError):
            return None
        if found is None:
            return None
        spec = importlib.util.spec_from_loader(fullname, _AliasLoader(real), is_package=found.submodule_search_locations is not None)
        return spec


if not any(isinstance(f, _AliasFinder) for f in sys.meta_path):
    sys.meta_path.insert(0, _AliasFinder())


def __getattr__(name: str):
    return getattr(_impl, name)


def __dir__():
    return __all__
