#!/usr/bin/env python
"""Cast a block-scaled fp8 checkpoint to bf16, file by file, keeping names and sharding.

    python toolkit/weight_convert/deepseekv3/fp8_cast_bf16.py --input-fp8-hf-path /hf/DeepSeek-V3 \\
        --output-bf16-hf-path /hf/DeepSeek-V3-bf16

Same job as the reference's ``research/deepseek3/fp8_cast_bf16.py`` (:31 ``weight_dequant``): every e4m3 ``X.weight``
is multiplied block by block (128 x 128) with its ``X.weight_scale_inv`` and written as bf16; the scale tensors are
dropped from the output and from ``model.safetensors.index.json``. A scale that lives in another shard than its weight
is fetched through the index. Only needed for consumers without an fp8 path: this framework loads the fp8 files
directly (``load_checkpoint`` / ``WeightsLoader`` with ``keep_fp8``).
"""
import argparse
import json
import os
import shutil
import sys

import torch
from safetensors.torch import load_file, save_file

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
sys.path.insert(0, ROOT)

from mindformers_b200.checkpoint.name_maps import weight_dequant  # noqa: E402
from mindformers_b200.inference.weights_utils import WeightsLoader  # noqa: E402


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--input-fp8-hf-path", required=True)
    ap.add_argument("--output-bf16-hf-path", required=True)
    a = ap.parse_args(argv)
    src, dst = a.input_fp8_hf_path, a.output_bf16_hf_path
    os.makedirs(dst, exist_ok=True)
    loader = WeightsLoader(src)
    weight_map, cast = {}, 0
    for path in loader.files:
        fname = os.path.basename(path)
        out = {}
        for name, t in load_file(path).items():
            if name.endswith("_scale_inv"):
                continue
            if t.dtype == torch.float8_e4m3fn:
                scale_name = name + "_scale_inv"
                if not loader.has(scale_name):
                    raise KeyError(f"{name} is fp8 but {scale_name} is nowhere in {src}")
                t = weight_dequant(t, loader.get(scale_name)).to(torch.bfloat16)
                cast += 1
            out[name] = t.contiguous()
            weight_map[name] = fname
        save_file(out, os.path.join(dst, fname), metadata={"format": "pt"})
    loader.close()
    total = 0
    for fname in sorted(set(weight_map.values())):
        total += os.path.getsize(os.path.join(dst, fname))
    with open(os.path.join(dst, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {"total_size": total}, "weight_map": weight_map}, f, indent=1)
    for extra in os.listdir(src):                       # config, tokenizer files
        if not extra.endswith(".safetensors") and not extra.endswith(".safetensors.index.json"):
            p = os.path.join(src, extra)
            if os.path.isfile(p):
                shutil.copy(p, os.path.join(dst, extra))
    cfg_file = os.path.join(dst, "config.json")
    if os.path.exists(cfg_file):
        cfg = json.load(open(cfg_file))
        if cfg.pop("quantization_config", None) is not None:
            json.dump(cfg, open(cfg_file, "w"), indent=1)
    print(f"cast {cast} fp8 tensors to bf16 into {dst}")
    return dst


if __name__ == "__main__":
    main()
