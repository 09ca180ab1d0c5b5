#!/usr/bin/env python
"""Merge per-rank safetensors checkpoints and their strategy files into one full checkpoint.

    python toolkit/safetensors/unified_safetensors.py --src_strategy_dirs output/strategy \
        --mindspore_ckpt_dir output/checkpoint --output_dir output/unified_checkpoint

Flags follow the reference's ``toolkit/safetensors/unified_safetensors.py:31,54``; the work is done by
``mindformers_b200.checkpoint.transform.unify_checkpoints`` (merge shards by the JSON strategy, write
``hyper_param.safetensors`` for the optimizer state).
"""
import argparse
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from mindformers_b200.checkpoint.transform import unify_checkpoints  # noqa: E402


def main(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("--src_strategy_dirs", required=True)
    p.add_argument("--mindspore_ckpt_dir", "--ckpt_dir", dest="ckpt_dir", required=True)
    p.add_argument("--output_dir", required=True)
    p.add_argument("--file_suffix", default=None, help="<epoch>_<step> of the checkpoint to merge (default: latest)")
    p.add_argument("--has_redundancy", default="True")
    p.add_argument("--filter_out_param_prefix", default=None)
    p.add_argument("--max_process_num", type=int, default=1)
    args = p.parse_args(argv)
    out = unify_checkpoints(args.ckpt_dir, args.src_strategy_dirs, args.output_dir, include_optimizer=args.filter_out_param_prefix is None)
    print(f"unified checkpoint written to {out}")
    return out


if __name__ == "__main__":
    main()
