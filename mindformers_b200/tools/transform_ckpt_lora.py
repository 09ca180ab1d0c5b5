"""Fold LoRA weights of a fine-tuned checkpoint into the base weights.

    python -m mindformers_b200.tools.transform_ckpt_lora --src_ckpt_path_or_dir ckpt/ --dst_ckpt_dir merged/ \\
        --lora_scaling 2.0 [--prefix checkpoint_] [--save_format safetensors]

For every pair ``X.lora_a [r, in]`` / ``X.lora_b [out, r]`` (this package's names; the reference's
``X.mindpet_delta_lora_a`` / ``…_b`` are accepted too) the base weight ``X.base.weight`` (or ``X.weight``) becomes
``W + scaling · B A`` and the pair is dropped; the result loads into a model built without LoRA. ``lora_scaling`` is
``lora_alpha / lora_rank``. Sharded inputs (several ``*.safetensors`` files or ``rank_N`` directories) are read
together; resharding between parallel layouts is the job of ``checkpoint.transform`` and runs before or after.

Reference: ``mindformers/tools/transform_ckpt_lora.py`` (argument names ``:64-95``; the merge ``W + scaling·BA``).
"""
from __future__ import annotations

import argparse
import glob
import os
from typing import Dict, Tuple

import torch

A_SUFFIXES = (".lora_a", ".mindpet_delta_lora_a")
B_SUFFIXES = (".lora_b", ".mindpet_delta_lora_b")


def merge_lora_state(state: Dict[str, torch.Tensor], scaling: float, fan_in_fan_out: bool = False
                     ) -> Tuple[Dict[str, torch.Tensor], int]:
    """Returns ``(merged state, number of merged layers)``."""
    out: Dict[str, torch.Tensor] = {}
    pairs: Dict[str, Dict[str, torch.Tensor]] = {}
    for name, t in state.items():
        for sfx in A_SUFFIXES:
            if name.endswith(sfx):
                pairs.setdefault(name[:-len(sfx)], {})["a"] = t
                break
        else:
            for sfx in B_SUFFIXES:
                if name.endswith(sfx):
                    pairs.setdefault(name[:-len(sfx)], {})["b"] = t
                    break
            else:
                out[name] = t
    merged = 0
    for prefix, ab in pairs.items():
        if "a" not in ab or "b" not in ab:
            raise KeyError(f"{prefix}: found only one of lora_a / lora_b")
        base_name = next((n for n in (prefix + ".base.weight", prefix + ".weight") if n in out), None)
        if base_name is None:
            raise KeyError(f"{prefix}: no base weight ({prefix}.base.weight or {prefix}.weight) in the checkpoint")
        w = out.pop(base_name)
        delta = ab["b"].float() @ ab["a"].float() * scaling
        if fan_in_fan_out:
            delta = delta.t()
        if delta.shape != w.shape:
            raise ValueError(f"{prefix}: B·A has shape {tuple(delta.shape)}, base weight {tuple(w.shape)}")
        out[prefix + ".weight"] = (w.float() + delta).to(w.dtype)
        bias = out.pop(prefix + ".base.bias", None)
        if bias is not None:
            out[prefix + ".bias"] = bias
        merged += 1
    return out, merged


def _collect(path: str):
    if os.path.isfile(path):
        return [path]
    files = sorted(glob.glob(os.path.join(path, "*.safetensors"))) or sorted(
        glob.glob(os.path.join(path, "rank_*", "*.safetensors")))
    if not files:
        raise FileNotFoundError(f"no .safetensors files under {path}")
    return files


def main(argv=None):
    from safetensors.torch import load_file, save_file
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--src_ckpt_strategy", default=None, help="accepted for command-line parity; layouts are read from the files")
    p.add_argument("--dst_ckpt_strategy", default=None, help="accepted for command-line parity")
    p.add_argument("--src_ckpt_path_or_dir", required=True)
    p.add_argument("--dst_ckpt_dir", required=True)
    p.add_argument("--prefix", default="checkpoint_")
    p.add_argument("--lora_scaling", type=float, default=1.0)
    p.add_argument("--fan_in_fan_out", action="store_true")
    p.add_argument("--save_format", default="safetensors", choices=["safetensors"])
    args = p.parse_args(argv)
    files = _collect(args.src_ckpt_path_or_dir)
    by_dir: Dict[str, Dict[str, torch.Tensor]] = {}
    for f in files:
        by_dir.setdefault(os.path.dirname(f), {}).update(load_file(f))
    total = 0
    for i, (src_dir, state) in enumerate(sorted(by_dir.items())):
        merged, n = merge_lora_state(state, args.lora_scaling, args.fan_in_fan_out)
        total += n
        sub = os.path.basename(src_dir) if os.path.basename(src_dir).startswith("rank_") else ""
        dst = os.path.join(args.dst_ckpt_dir, sub)
        os.makedirs(dst, exist_ok=True)
        save_file({k: v.contiguous() for k, v in merged.items()}, os.path.join(dst, f"{args.prefix}{i}.safetensors"))
    print(f"merged {total} LoRA layers from {len(files)} file(s) into {args.dst_ckpt_dir}")
    return total


if __name__ == "__main__":
    main()
