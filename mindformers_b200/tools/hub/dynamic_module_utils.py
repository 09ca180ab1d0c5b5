"""Loading model / tokenizer classes from Python files that ship inside a model directory (``auto_map``) or live
under ``$REGISTER_PATH``.

Reference: ``mindformers/tools/hub/dynamic_module_utils.py`` (``get_class_from_dynamic_module``,
``get_class_in_module``, ``check_imports``) and the ``--register_path`` flag of ``run_mindformer.py:225-231``.
A reference ``"file_name.ClassName"`` names a file of the directory; its relative imports (``from .other import X``)
are resolved against the same directory by loading the directory as a throw-away package.
"""
from __future__ import annotations

import hashlib
import importlib
import importlib.util
import os
import re
import sys
from typing import List, Optional, Type

_PKG_PREFIX = "mfb200_dynamic_"


def get_relative_imports(module_file: str) -> List[str]:
    """Names ``x`` of every ``from .x import`` / ``import .x`` of the file."""
    with open(module_file, "r", encoding="utf-8") as f:
        src = f.read()
    rel = re.findall(r"^\s*from\s+\.(\w+)\s+import", src, flags=re.MULTILINE)
    rel += re.findall(r"^\s*import\s+\.(\w+)", src, flags=re.MULTILINE)
    return sorted(set(rel))


def get_imports(module_file: str) -> List[str]:
    """Top-level packages the file imports (relative imports and ``try:`` guarded ones left out)."""
    with open(module_file, "r", encoding="utf-8") as f:
        src = f.read()
    src = re.sub(r"\s*try\s*:.*?except.*?:", "", src, flags=re.DOTALL)
    mods = re.findall(r"^\s*import\s+(\S+)", src, flags=re.MULTILINE)
    mods += re.findall(r"^\s*from\s+(\S+)\s+import", src, flags=re.MULTILINE)
    return sorted({m.split(".")[0] for m in mods if not m.startswith(".")})


def check_imports(module_file: str) -> List[str]:
    """Raise ``ImportError`` naming every package the file needs that is not installed; returns its relative imports."""
    missing = []
    for name in get_imports(module_file):
        if name and importlib.util.find_spec(name) is None:
            missing.append(name)
    if missing:
        raise ImportError(f"{module_file} needs packages that are not installed: {', '.join(missing)}")
    return get_relative_imports(module_file)


def _package_for(directory: str) -> str:
    """Register ``directory`` as a package (once) and return its name."""
    directory = os.path.abspath(directory)
    name = _PKG_PREFIX + hashlib.sha1(directory.encode()).hexdigest()[:12]
    if name not in sys.modules:
        spec = importlib.machinery.ModuleSpec(name, loader=None, is_package=True)
        pkg = importlib.util.module_from_spec(spec)
        pkg.__path__ = [directory]
        sys.modules[name] = pkg
    return name


def get_class_in_module(class_name: str, module_file: str, force_reload: bool = False) -> Type:
    """Import ``module_file`` (as a member of its directory's package) and return its attribute ``class_name``."""
    directory, fname = os.path.split(os.path.abspath(module_file))
    pkg = _package_for(directory)
    mod_name = f"{pkg}.{os.path.splitext(fname)[0]}"
    if force_reload:
        sys.modules.pop(mod_name, None)
    module = sys.modules.get(mod_name) or importlib.import_module(mod_name)
    if not hasattr(module, class_name):
        raise AttributeError(f"{module_file} defines no {class_name}")
    return getattr(module, class_name)


def get_class_from_dynamic_module(class_reference: str, pretrained_model_name_or_path: str,
                                  force_reload: bool = False, **kwargs) -> Type:
    """``class_reference`` = ``"modeling_x.MyModel"`` (optionally ``"repo--modeling_x.MyModel"``): the class of that
    file in the model directory."""
    if "--" in class_reference:
        _, class_reference = class_reference.split("--", 1)
    module_name, class_name = class_reference.rsplit(".", 1)
    module_file = os.path.join(pretrained_model_name_or_path, module_name.replace(".", os.sep) + ".py")
    if not os.path.isfile(module_file):
        raise FileNotFoundError(f"{module_file} (from auto_map entry {class_reference!r}) does not exist")
    for rel in check_imports(module_file):
        dep = os.path.join(os.path.dirname(module_file), rel + ".py")
        if not os.path.isfile(dep) and not os.path.isdir(os.path.join(os.path.dirname(module_file), rel)):
            raise FileNotFoundError(f"{module_file} imports .{rel}, which is missing from the directory")
    return get_class_in_module(class_name, module_file, force_reload)


def import_register_path(path: Optional[str] = None) -> List[str]:
    """Import every ``*.py`` of ``path`` (default ``$REGISTER_PATH``) so that their ``@MindFormerRegister.register``
    decorators run; returns the imported module names."""
    path = path or os.environ.get("REGISTER_PATH")
    if not path:
        return []
    if not os.path.isdir(path):
        raise NotADirectoryError(f"REGISTER_PATH {path} is not a directory")
    done = []
    for fname in sorted(os.listdir(path)):
        if fname.endswith(".py") and not fname.startswith("_"):
            pkg = _package_for(path)
            name = f"{pkg}.{fname[:-3]}"
            if name not in sys.modules:
                importlib.import_module(name)
            done.append(name)
    return done
