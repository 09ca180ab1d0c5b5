#!/usr/bin/env python
"""Instruction data (json / jsonl, or a Hugging Face ``datasets`` directory when that package is present) → tokenised,
optionally packed samples saved as ``.npz`` shards that ``CommonDataLoader`` reads.

    python toolkit/data_preprocess/huggingface/datasets_preprocess.py --input alpaca.json --handler AlpacaInstructDataHandler \
        --seq-length 4096 --pack --output out/alpaca_packed

Reference: ``toolkit/data_preprocess/huggingface/datasets_preprocess.py:28,88`` (config-driven handlers + packing).
"""
import argparse
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
sys.path.insert(0, ROOT)

from mindformers_b200.dataset.handlers import PackingHandler, build_data_handler  # noqa: E402
from mindformers_b200.models import build_tokenizer  # noqa: E402


def read_records(path):
    if os.path.isdir(path):
        try:
            import datasets
            return list(datasets.load_from_disk(path))
        except ImportError as e:
            raise SystemExit("reading a datasets directory needs the `datasets` package; pass a json/jsonl file") from e
    with open(path, encoding="utf-8") as f:
        text = f.read().strip()
    if text.startswith("["):
        return json.loads(text)
    return [json.loads(line) for line in text.splitlines() if line.strip()]


def main(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("--input", required=True)
    p.add_argument("--output", required=True)
    p.add_argument("--handler", default="AlpacaInstructDataHandler")
    p.add_argument("--tokenizer-type", default="ByteTokenizer")
    p.add_argument("--tokenizer-dir", default=None)
    p.add_argument("--seq-length", type=int, default=2048)
    p.add_argument("--pack", action="store_true")
    p.add_argument("--shard-size", type=int, default=10000)
    args = p.parse_args(argv)
    tok = build_tokenizer({"type": "AutoTokenizer", "pretrained_model_name_or_path": args.tokenizer_dir} if args.tokenizer_dir
                          else {"type": args.tokenizer_type})
    handler = build_data_handler({"type": args.handler, "tokenizer": tok, "seq_length": args.seq_length, "padding": not args.pack})
    samples = handler.handle(read_records(args.input))
    if args.pack:
        samples = PackingHandler(args.seq_length, pad_token_id=getattr(tok, "pad_token_id", 0) or 0).handle(samples)
    os.makedirs(os.path.dirname(os.path.abspath(args.output)) or ".", exist_ok=True)
    n = 0
    for i in range(0, len(samples), args.shard_size):
        chunk = samples[i:i + args.shard_size]
        keys = chunk[0].keys()
        np.savez(f"{args.output}_{i // args.shard_size:05d}.npz", **{k: np.stack([np.asarray(s[k]) for s in chunk]) for k in keys})
        n += len(chunk)
    print(f"wrote {n} samples of length {args.seq_length} to {args.output}_*.npz")
    return n


if __name__ == "__main__":
    main()
