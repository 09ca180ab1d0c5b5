"""Command line of the offline checkpoint transformation (reference ``mindformers/tools/transform_ckpt.py``).

    python -m mindformers_b200.tools.transform_ckpt --src_ckpt_dir output/checkpoint --src_ckpt_strategy output/strategy \\
        --dst_ckpt_strategy other/strategy --dst_ckpt_dir transformed --prefix llama_
"""
from __future__ import annotations

import argparse

from .ckpt_transform import TransformCkpt


def main(argv=None):
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--src_ckpt_strategy", default=None, help="directory of the source layout's strategy files (omit for a complete checkpoint)")
    p.add_argument("--dst_ckpt_strategy", default=None, help="directory of the destination layout's strategy files (omit to merge only)")
    p.add_argument("--src_ckpt_dir", required=True)
    p.add_argument("--dst_ckpt_dir", required=True)
    p.add_argument("--prefix", default="checkpoint_")
    p.add_argument("--no_optimizer", action="store_true", help="drop the optimizer states")
    p.add_argument("--rank_id", type=int, default=None, help="with --world_size: this process converts the destination ranks r % world_size == rank_id")
    p.add_argument("--world_size", type=int, default=None)
    a = p.parse_args(argv)
    out = TransformCkpt(include_optimizer=not a.no_optimizer, rank_id=a.rank_id, world_size=a.world_size)(
        a.src_ckpt_dir, a.dst_ckpt_dir, a.src_ckpt_strategy, a.dst_ckpt_strategy, a.prefix)
    print(out)
    return out


if __name__ == "__main__":
    main()
