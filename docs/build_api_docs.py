#!/usr/bin/env python
"""Write the API reference under ``docs/api`` from the docstrings of the public packages (the reference ships a
hand-written ``docs/api`` tree; here the docstrings are the single source and this script renders them):

    python docs/build_api_docs.py            # rewrites docs/api/*.md
    python docs/build_api_docs.py --check    # exit 1 when the files on disk are stale (used by the test suite)

One page per package: its module docstring, then every public class (with its public methods) and function with
signature and docstring, in source order."""
import argparse
import importlib
import inspect
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

PACKAGES = [
    "mindformers_b200", "mindformers_b200.core", "mindformers_b200.core.callback", "mindformers_b200.core.lr",
    "mindformers_b200.core.optim", "mindformers_b200.core.metric", "mindformers_b200.core.context",
    "mindformers_b200.models", "mindformers_b200.models.modeling_utils", "mindformers_b200.models.configuration_utils",
    "mindformers_b200.models.tokenization_utils", "mindformers_b200.generation", "mindformers_b200.pipeline",
    "mindformers_b200.trainer", "mindformers_b200.trainer.base_trainer", "mindformers_b200.trainer.engine",
    "mindformers_b200.dataset", "mindformers_b200.pet", "mindformers_b200.wrapper", "mindformers_b200.checkpoint.io",
    "mindformers_b200.checkpoint.transform", "mindformers_b200.parallel.parallel_state",
    "mindformers_b200.parallel.transformer_config", "mindformers_b200.parallel.pipeline",
    "mindformers_b200.parallel.ring_attention", "mindformers_b200.parallel.recompute",
    "mindformers_b200.parallel.layers.attention", "mindformers_b200.parallel.layers.moe",
    "mindformers_b200.parallel.layers.moe_dispatchers", "mindformers_b200.parallel.layers.tensor_parallel",
    "mindformers_b200.parallel.layers.gpt_model", "mindformers_b200.parallel.distributed.optimizer",
    "mindformers_b200.inference.paged_attention", "mindformers_b200.serving.engine", "mindformers_b200.serving.api_server",
    "mindformers_b200.ops.functional", "mindformers_b200.ops.attention", "mindformers_b200.tools.register",
    "mindformers_b200.tools.check_rules", "mindformers_b200.modules.quantizers", "mindformers_b200.modules.seq_pipe",
    "mindformers_b200.model_runner",
]


def _sig(obj) -> str:
    try:
        return str(inspect.signature(obj))
    except (TypeError, ValueError):
        return "(...)"


def _doc(obj) -> str:
    return inspect.cleandoc(getattr(obj, "__doc__", None) or "").strip()


def _members(mod):
    names = getattr(mod, "__all__", None)
    if names is None:
        names = [n for n, o in vars(mod).items() if not n.startswith("_")
                 and (inspect.isclass(o) or inspect.isfunction(o)) and getattr(o, "__module__", "").startswith(mod.__name__)]
    out = []
    for n in names:
        try:
            o = getattr(mod, n)
        except Exception:   # noqa: BLE001
            continue
        if inspect.isclass(o) or inspect.isfunction(o):
            out.append((n, o))

    def line_of(item):
        try:
            return (inspect.getsourcefile(item[1]) or "", inspect.getsourcelines(item[1])[1])
        except (OSError, TypeError):
            return ("", 0)
    return sorted(out, key=line_of)


def render(module_name: str) -> str:
    mod = importlib.import_module(module_name)
    lines = [f"# `{module_name}`", ""]
    if _doc(mod):
        lines += [_doc(mod), ""]
    for name, obj in _members(mod):
        if inspect.isclass(obj):
            lines += [f"## class `{name}{_sig(obj)}`", ""]
            if _doc(obj):
                lines += [_doc(obj), ""]
            for mname, meth in vars(obj).items():
                if mname.startswith("_") or not (inspect.isfunction(meth) or isinstance(meth, (classmethod, staticmethod))):
                    continue
                fn = meth.__func__ if isinstance(meth, (classmethod, staticmethod)) else meth
                if not _doc(fn):
                    continue
                lines += [f"### `{name}.{mname}{_sig(fn)}`", "", _doc(fn), ""]
        else:
            lines += [f"## `{name}{_sig(obj)}`", ""]
            if _doc(obj):
                lines += [_doc(obj), ""]
    return "\n".join(lines).rstrip() + "\n"


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--check", action="store_true")
    args = ap.parse_args(argv)
    out_dir = os.path.join(ROOT, "docs", "api")
    os.makedirs(out_dir, exist_ok=True)
    stale = []
    index = ["# API reference", "", "Generated from the docstrings by `python docs/build_api_docs.py`.", ""]
    for name in PACKAGES:
        text = render(name)
        path = os.path.join(out_dir, name + ".md")
        index.append(f"* [`{name}`]({name}.md)")
        if args.check:
            if not os.path.exists(path) or open(path, encoding="utf-8").read() != text:
                stale.append(name)
        else:
            with open(path, "w", encoding="utf-8") as f:
                f.write(text)
    idx_text = "\n".join(index) + "\n"
    idx_path = os.path.join(out_dir, "README.md")
    if args.check:
        if not os.path.exists(idx_path) or open(idx_path, encoding="utf-8").read() != idx_text:
            stale.append("README")
        if stale:
            print("stale API pages:", ", ".join(stale))
            return 1
        return 0
    with open(idx_path, "w", encoding="utf-8") as f:
        f.write(idx_text)
    print(f"wrote {len(PACKAGES)} pages to {out_dir}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
