"""YAML-backed configuration tree.

``MindFormerConfig`` is a ``dict`` whose keys are also attributes (missing attributes read as
``None``), loadable from YAML files with ``base_config:`` inheritance, and updatable with dotted keys
(``runner_config.batch_size=4``). It mirrors the behaviour of the reference's
``mindformers/tools/register/config.py`` (``MindFormerConfig`` :75, ``_file2dict`` :171-208,
``merge_from_dict`` :122-148, ``ActionDict`` :304-401) without sharing its implementation.
"""
from __future__ import annotations

import argparse
import ast
import copy
import os
from typing import Any, Iterable

import yaml

BASE_KEY = "base_config"
MAX_YAML_DEPTH = 10


def _wrap(value):
    if isinstance(value, MindFormerConfig):
        return value
    if isinstance(value, dict):
        return MindFormerConfig(**value)
    if isinstance(value, (list, tuple)):
        return type(value)(_wrap(v) for v in value)
    return value


def _depth(obj, level=0):
    if level > MAX_YAML_DEPTH:
        raise ValueError(f"configuration nesting deeper than {MAX_YAML_DEPTH} levels")
    if isinstance(obj, dict):
        for v in obj.values():
            _depth(v, level + 1)
    elif isinstance(obj, (list, tuple)):
        for v in obj:
            _depth(v, level + 1)


class DictConfig(dict):
    """A dict whose keys are also attributes (reference ``tools/register/config.py:31``); missing attributes read None.
    ``to_dict`` gives back plain nested dicts."""

    def __getattr__(self, key):
        return self.get(key)

    def __setattr__(self, key, value):
        self[key] = value

    def __delattr__(self, key):
        del self[key]

    def __deepcopy__(self, memo=None):
        out = DictConfig()
        for k, v in self.items():
            out[copy.deepcopy(k, memo)] = copy.deepcopy(v, memo)
        return out

    def to_dict(self):
        out = {}
        for k, v in self.items():
            out[k] = v.to_dict() if isinstance(v, DictConfig) else copy.deepcopy(v)
        return out


class MindFormerConfig(dict):
    """Nested attribute dictionary. ``MindFormerConfig("a.yaml", "b.yaml", key=value)``."""

    def __init__(self, *args, **kwargs):
        super().__init__()
        merged: dict = {}
        for arg in args:
            if isinstance(arg, str):
                if not arg.endswith((".yaml", ".yml")):
                    raise ValueError(f"configuration file must be YAML, got {arg!r}")
                _deep_update(merged, self._file2dict(arg))
            elif isinstance(arg, dict):
                _deep_update(merged, arg)
            elif arg is not None:
                raise TypeError(f"unsupported configuration source {type(arg).__name__}")
        _deep_update(merged, kwargs)
        for k, v in merged.items():
            dict.__setitem__(self, k, _wrap(v))

    # ---- attribute protocol ------------------------------------------------------------------
    def __getattr__(self, key):
        if key.startswith("__"):
            raise AttributeError(key)
        return self.get(key)

    def __setattr__(self, key, value):
        dict.__setitem__(self, key, _wrap(value))

    def __setitem__(self, key, value):
        dict.__setitem__(self, key, _wrap(value))

    def __delattr__(self, key):
        if key in self:
            del self[key]

    def __deepcopy__(self, memo):
        out = MindFormerConfig()
        for k, v in self.items():
            dict.__setitem__(out, copy.deepcopy(k, memo), copy.deepcopy(v, memo))
        return out

    # ---- loading -------------------------------------------------------------------------------
    @staticmethod
    def _file2dict(filename: str, _seen: tuple = ()) -> dict:
        path = os.path.realpath(os.path.expanduser(filename))
        if not os.path.isfile(path):
            raise FileNotFoundError(f"configuration file {filename} not found")
        if path in _seen:
            raise ValueError(f"circular base_config chain through {filename}")
        with open(path, encoding="utf-8") as f:
            text = f.read()
        from ..check_rules import check_yaml_depth_before_loading
        check_yaml_depth_before_loading(text)          # on the node tree, before any object is built
        data = yaml.safe_load(text) or {}
        if not isinstance(data, dict):
            raise ValueError(f"{filename}: top level of a configuration must be a mapping")
        _depth(data)
        result: dict = {}
        bases = data.pop(BASE_KEY, None)
        if bases:
            if isinstance(bases, str):
                bases = [bases]
            for base in bases:
                base_path = base if os.path.isabs(base) else os.path.join(os.path.dirname(path), base)
                _deep_update(result, MindFormerConfig._file2dict(base_path, _seen + (path,)))
        _deep_update(result, data)
        return result

    # ---- updates -------------------------------------------------------------------------------
    def merge_from_dict(self, options: dict):
        """Update from ``{"a.b.c": value}`` style options (plain nested dicts work too)."""
        for full_key, value in options.items():
            parts = full_key.split(".")
            node = self
            for part in parts[:-1]:
                nxt = node.get(part)
                if not isinstance(nxt, dict):
                    nxt = MindFormerConfig()
                    node[part] = nxt
                node = node[part]
            last = parts[-1]
            if isinstance(value, dict) and isinstance(node.get(last), dict):
                node[last].merge_from_dict(value)
            else:
                node[last] = value

    def get_value(self, key, default=None):
        """``cfg.get_value("a.b")`` or ``cfg.get_value(["a", "b"])``."""
        parts = key.split(".") if isinstance(key, str) else list(key)
        node: Any = self
        for part in parts:
            if not isinstance(node, dict) or part not in node:
                return default
            node = node[part]
        return node

    def set_value(self, key, value):
        parts = key.split(".") if isinstance(key, str) else list(key)
        self.merge_from_dict({".".join(parts): value})

    def to_dict(self) -> dict:
        def unwrap(v):
            if isinstance(v, dict):
                return {k: unwrap(x) for k, x in v.items()}
            if isinstance(v, (list, tuple)):
                return type(v)(unwrap(x) for x in v)
            return v
        return unwrap(self)

    def dump(self, path: str):
        with open(path, "w", encoding="utf-8") as f:
            yaml.safe_dump(self.to_dict(), f, sort_keys=False)


def _deep_update(dst: dict, src: dict):
    for k, v in src.items():
        if isinstance(v, dict) and isinstance(dst.get(k), dict):
            _deep_update(dst[k], v)
        else:
            dst[k] = copy.deepcopy(v) if isinstance(v, (dict, list)) else v


def parse_value(text: str):
    """Literal parsing of a command-line value: numbers, booleans, None, lists, dicts, else string."""
    low = text.strip()
    if low.lower() in ("true", "false"):
        return low.lower() == "true"
    if low.lower() in ("none", "null"):
        return None
    try:
        return ast.literal_eval(low)
    except (ValueError, SyntaxError):
        return text


class ActionDict(argparse.Action):
    """``--options a.b=1 c=[1,2]`` → ``{"a.b": 1, "c": [1, 2]}``."""

    def __call__(self, parser, namespace, values: Iterable[str], option_string=None):
        options = getattr(namespace, self.dest, None) or {}
        for item in values:
            if "=" not in item:
                raise argparse.ArgumentError(self, f"expected key=value, got {item!r}")
            key, val = item.split("=", 1)
            options[key.strip()] = parse_value(val)
        setattr(namespace, self.dest, options)
