#!/usr/bin/env python
"""Hugging Face ⇄ framework weight converter.

    python convert_weight.py --model llama --input_path /hf/dir_or_file --output_path out.safetensors [--dtype bf16]
    python convert_weight.py --model qwen2_5 --reversed --input_path ckpt.safetensors --output_path hf_dir

``--model`` picks the name map (the reference's table in ``convert_weight.py:36-49``: llama, qwen2_5, glm-n,
mixtral, telechat, deepseekv3; plus qwen3 / qwen3_moe here). ``--qkv_concat`` is the default and only layout the
networks own (``linear_qkv`` / ``linear_fc1`` fused); ``--legacy_names`` writes the older
``model.layers.N.attention.wq`` style names instead. DeepSeek-V3 fp8 checkpoints (``weight_scale_inv`` blocks of
128×128) are dequantised to the target dtype, or kept in fp8 with their scales by ``--keep_fp8``.
"""
import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402
from safetensors.torch import load_file, save_file  # noqa: E402

from mindformers_b200.checkpoint import name_maps  # noqa: E402
from mindformers_b200.checkpoint.io import resolve_checkpoint  # noqa: E402
from mindformers_b200.models.auto import AutoConfig  # noqa: E402
from mindformers_b200.models.presets import preset_is_mla  # noqa: E402
from mindformers_b200.parallel.transformer_config_utils import convert_to_transformer_config  # noqa: E402

convert_map = {"llama": "llama", "qwen2_5": "qwen2", "qwen2": "qwen2", "qwen3": "qwen3", "qwen3_moe": "qwen3_moe",
               "glm-n": "glm", "glm4": "glm", "mixtral": "mixtral", "telechat": "telechat", "deepseekv3": "deepseek_v3",
               "deepseekv2": "deepseek_v2", "qwen2_moe": "qwen2_moe"}
reversed_convert_map = dict(convert_map)
DTYPES = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16}


def _load_any(path):
    if os.path.isdir(path):
        _, files = resolve_checkpoint(path)
    else:
        files = [path]
    sd = {}
    for f in files:
        if f.endswith(".safetensors"):
            sd.update(load_file(f))
        else:
            sd.update(torch.load(f, map_location="cpu", weights_only=True))
    return sd


def _config_for(args, input_dir):
    cfg_path = args.config or (os.path.join(input_dir, "config.json") if os.path.isdir(input_dir) else None)
    if not cfg_path or not os.path.exists(cfg_path):
        raise SystemExit("a model configuration is needed for the fused layouts: pass --config config.json")
    with open(cfg_path) as f:
        d = json.load(f)
    d.setdefault("model_type", convert_map[args.model])
    return convert_to_transformer_config(d, is_mla_model=preset_is_mla(d), strict=False)


def convert(args):
    family = convert_map[args.model]
    dtype = DTYPES[args.dtype] if args.dtype else None
    if args.workers and args.workers > 1 and not args.reversed and not args.legacy_names and os.path.isdir(args.input_path):
        # one process per group of layers, one output file each + an index (a directory, not a single file)
        from mindformers_b200.utils.safetensors import convert_hf_safetensors_multiprocess
        cfg_path = args.config or os.path.join(args.input_path, "config.json")
        with open(cfg_path) as f:
            cfg_dict = json.load(f)
        cfg_dict.setdefault("model_type", family)
        return convert_hf_safetensors_multiprocess(args.input_path, args.output_path, cfg_dict, family,
                                                   {"fp32": "float32", "bf16": "bfloat16", "fp16": "float16"}.get(args.dtype),
                                                   workers=args.workers, keep_fp8=args.keep_fp8)
    sd = _load_any(args.input_path)
    cfg = _config_for(args, args.input_path)
    if args.reversed:
        out = name_maps.framework_to_hf(sd, cfg, family, dtype)
        os.makedirs(args.output_path, exist_ok=True)
        save_file(out, os.path.join(args.output_path, "model.safetensors"), metadata={"format": "pt"})
        return os.path.join(args.output_path, "model.safetensors")
    if args.legacy_names:
        out = {name_maps.convert_name_legacy(k): (v.to(dtype) if dtype is not None and v.is_floating_point() else v)
               for k, v in sd.items() if "rotary_emb.inv_freq" not in k}
    else:
        out = name_maps.hf_to_framework(sd, cfg, family, dtype, keep_fp8=args.keep_fp8)
    out = {k: v.contiguous() for k, v in out.items()}
    os.makedirs(os.path.dirname(os.path.abspath(args.output_path)) or ".", exist_ok=True)
    path = args.output_path if args.output_path.endswith(".safetensors") else args.output_path + ".safetensors"
    save_file(out, path, metadata={"format": "pt"})
    return path


def main(argv=None):
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--model", required=True, choices=sorted(convert_map))
    p.add_argument("--reversed", action="store_true", help="framework → Hugging Face")
    p.add_argument("--input_path", default=None)
    p.add_argument("--output_path", default=None)
    p.add_argument("--convert_config", default=None,
                   help="YAML with one section per model (input_path, output_path, dtype, ...), e.g. "
                        "configs/convert_config/run_convert.yaml; command-line values win")
    p.add_argument("--dtype", default=None, choices=sorted(DTYPES))
    p.add_argument("--config", default=None, help="config.json of the model (defaults to <input_path>/config.json)")
    p.add_argument("--qkv_concat", default=True, type=lambda s: s.lower() in ("1", "true"))
    p.add_argument("--legacy_names", action="store_true")
    p.add_argument("--keep_fp8", action="store_true")
    p.add_argument("--workers", type=int, default=1,
                   help="> 1: convert a Hugging Face directory with this many processes (output_path becomes a directory "
                        "of files + model.safetensors.index.json)")
    p.add_argument("--n_head", type=int, default=None)
    p.add_argument("--hidden_size", type=int, default=None)
    p.add_argument("--layers", type=int, default=None)
    args = p.parse_args(argv)
    if args.convert_config:
        import yaml
        with open(args.convert_config) as f:
            section = (yaml.safe_load(f) or {}).get(args.model) or {}
        for key, value in section.items():
            if value is not None and hasattr(args, key) and getattr(args, key) in (None, False):
                setattr(args, key, value)
    if not args.input_path or not args.output_path:
        p.error("--input_path and --output_path are required (on the command line or in --convert_config)")
    path = convert(args)
    print(f"converted weights written to {path}")
    return path


if __name__ == "__main__":
    main()
