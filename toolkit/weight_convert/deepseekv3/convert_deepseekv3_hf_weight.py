#!/usr/bin/env python
"""DeepSeek-V3 Hugging Face checkpoint → this framework's parameter names and fused layouts.

    python toolkit/weight_convert/deepseekv3/convert_deepseekv3_hf_weight.py --torch_ckpt_path /hf/DeepSeek-V3 \
        --mindspore_ckpt_path out/dsv3 [--dtype bf16 | --keep_fp8] [--num_layers 61] [--worker_num 4]

What it does (same transformations as the reference tool, ``toolkit/weight_convert/deepseekv3/
convert_deepseekv3_hf_weight.py``: ``weight_dequant`` :67-114, attention map :219-310, MLP / MoE map :313-435, MTP
:438-506): fp8 ``weight`` + ``weight_scale_inv`` (128 x 128 blocks) are de-quantised to the target dtype, or kept in
fp8 next to their scales with ``--keep_fp8`` (the block-scaled GEMM consumes them directly); ``q_a_proj`` and
``kv_a_proj_with_mqa`` become ``linear_qkv``; gate and up projections become ``linear_fc1``; routed experts are stacked
into ``experts.weight1 [E, H, 2F]`` / ``experts.weight2 [E, F, H]``; the next-token-prediction layer goes to ``mtp.*``.
Files are converted one by one so that the host never holds more than a shard plus the tensors waiting for their partners.
"""
import argparse
import json
import os
import sys

import torch
from safetensors.torch import save_file

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
sys.path.insert(0, ROOT)

from mindformers_b200.checkpoint import name_maps  # noqa: E402
from mindformers_b200.parallel.transformer_config_utils import convert_to_transformer_config  # noqa: E402

DTYPES = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}


def n_main_full(hf_cfg) -> int:
    """Index of the first layer that is not a decoder layer of the full model (the MTP layers follow the decoder)."""
    return int(hf_cfg.get("num_hidden_layers_full", hf_cfg["num_hidden_layers"]))


def main(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("--torch_ckpt_path", required=True)
    p.add_argument("--mindspore_ckpt_path", required=True)
    p.add_argument("--dtype", default="bf16", choices=sorted(DTYPES))
    p.add_argument("--keep_fp8", action="store_true")
    p.add_argument("--num_layers", type=int, default=None, help="convert only the first N layers (plus embeddings, head and MTP)")
    p.add_argument("--use_grouped_gemm", default=True)
    p.add_argument("--worker_num", type=int, default=1)
    args = p.parse_args(argv)
    src, dst = args.torch_ckpt_path, args.mindspore_ckpt_path
    with open(os.path.join(src, "config.json")) as f:
        hf_cfg = json.load(f)
    if args.num_layers:
        hf_cfg["num_hidden_layers_full"] = hf_cfg["num_hidden_layers"]
        hf_cfg["num_hidden_layers"] = args.num_layers
    cfg = convert_to_transformer_config(hf_cfg, is_mla_model=True, strict=False)
    from mindformers_b200.inference.weights_utils import WeightsLoader
    loader = WeightsLoader(src)
    layers, other = loader.layer_groups()
    n_main = int(hf_cfg["num_hidden_layers"])
    os.makedirs(dst, exist_ok=True)
    shard, size, idx, index, total, count = {}, 0, 0, {}, 0, 0
    limit = 5 * (1 << 30)

    def flush():
        nonlocal shard, size, idx
        if shard:
            name = f"model-{idx:05d}.safetensors"
            save_file({k: v.contiguous() for k, v in shard.items()}, os.path.join(dst, name), metadata={"format": "pt"})
            for k in shard:
                index[k] = name
            shard, size, idx = {}, 0, idx + 1

    def emit(converted):
        nonlocal size, total, count
        for k, v in converted.items():
            nbytes = v.numel() * v.element_size()
            if size + nbytes > limit:
                flush()
            shard[k] = v
            size += nbytes
            total += nbytes
            count += 1

    # one group at a time: tensors outside the layers, then every layer (fused tensors have all their partners inside
    # their layer), so the host holds one layer of the source and one output shard at most
    groups = [sorted(other)]
    for i in sorted(layers):
        if args.num_layers and i >= args.num_layers and i < n_main_full(hf_cfg):
            continue                                   # a truncated conversion keeps the first N layers (and MTP)
        groups.append(sorted(layers[i]))
    for names in groups:
        if not names:
            continue
        part = loader.load_group(names)
        conv = name_maps.hf_to_framework(part, cfg, "deepseek_v3", DTYPES[args.dtype], keep_fp8=args.keep_fp8)
        if args.keep_fp8:
            for k, v in part.items():
                if k.endswith("_scale_inv"):
                    fw = name_maps.convert_name(k[:-len("_scale_inv")], "deepseek_v3") + "_scale_inv"
                    conv.setdefault(fw, v)
        emit(conv)
        del part, conv
    flush()
    loader.close()
    with open(os.path.join(dst, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {"total_size": total}, "weight_map": index}, f, indent=1)
    with open(os.path.join(dst, "config.json"), "w") as f:
        json.dump(hf_cfg, f, indent=1)
    print(f"converted {count} tensors into {dst}")
    return dst


if __name__ == "__main__":
    main()
