"""Optional-dependency probes and lazy module attributes (reference ``mindformers/utils/import_utils.py``)."""
from __future__ import annotations

import importlib
import importlib.util
import sys
from types import ModuleType
from typing import Dict, List


def is_package_available(name: str) -> bool:
    try:
        return importlib.util.find_spec(name) is not None
    except (ImportError, ValueError):
        return False


def is_tokenizers_available() -> bool:
    return is_package_available("tokenizers")


def is_sentencepiece_available() -> bool:
    return is_package_available("sentencepiece")


def is_tiktoken_available() -> bool:
    return is_package_available("tiktoken")


def is_jinja2_available() -> bool:
    return is_package_available("jinja2")


def is_pil_available() -> bool:
    return is_package_available("PIL")


def is_datasets_available() -> bool:
    return is_package_available("datasets")


def requires_backends(obj, backends: List[str]):
    """Raise ``ImportError`` naming the missing packages that ``obj`` needs."""
    missing = [b for b in backends if not is_package_available(b)]
    if missing:
        name = getattr(obj, "__name__", type(obj).__name__)
        raise ImportError(f"{name} needs the packages {missing}, which are not installed (no index access here)")


class LazyModule(ModuleType):
    """Module whose attributes are imported from sub-modules on first access: ``{"submodule": ["Name", …]}``."""

    def __init__(self, name: str, module_file: str, import_structure: Dict[str, List[str]]):
        super().__init__(name)
        self._structure = import_structure
        self._owner = {attr: mod for mod, attrs in import_structure.items() for attr in attrs}
        self.__file__ = module_file
        self.__path__ = [module_file.rsplit("/", 1)[0]]
        self.__all__ = list(self._owner) + list(import_structure)

    def __dir__(self):
        return sorted(set(super().__dir__()) | set(self.__all__))

    def __getattr__(self, attr: str):
        if attr in self._structure:
            value = importlib.import_module("." + attr, self.__name__)
        elif attr in self._owner:
            value = getattr(importlib.import_module("." + self._owner[attr], self.__name__), attr)
        else:
            raise AttributeError(f"module {self.__name__} has no attribute {attr}")
        setattr(self, attr, value)
        return value


def direct_import(name: str, path: str) -> ModuleType:
    """Import a file as module ``name`` regardless of ``sys.path``."""
    spec = importlib.util.spec_from_file_location(name, path)
    module = importlib.util.module_from_spec(spec)
    sys.modules[name] = module
    spec.loader.exec_module(module)
    return module
