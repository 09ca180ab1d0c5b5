#!/usr/bin/env python
"""json / jsonl text → Megatron indexed dataset (``<prefix>_<key>_document.bin/.idx``).

    python toolkit/data_preprocess/megatron/preprocess_indexed_dataset.py --input data.jsonl --output-prefix out/wiki \
        --tokenizer-type ByteTokenizer --json-keys text --append-eod --workers 4 --partitions 2

Counterpart of the reference's ``toolkit/data_preprocess/megatron/preprocess_indexed_dataset.py`` (``Encoder`` :47,
``Partition`` :110, ``main`` :377): the input is cut into ``--partitions`` line ranges, each encoded by a pool of
``--workers`` processes into its own index, and the partial indices are merged at the end.
"""
import argparse
import json
import multiprocessing
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
sys.path.insert(0, ROOT)

from mindformers_b200.dataset.indexed_dataset import IndexedDatasetBuilder, best_dtype, get_bin_path, get_idx_path  # noqa: E402


class Encoder:
    tokenizer = None

    def __init__(self, args):
        self.args = args

    def initializer(self):
        from mindformers_b200.models import build_tokenizer
        cfg = {"type": self.args.tokenizer_type}
        if self.args.tokenizer_dir:
            cfg = {"type": "AutoTokenizer", "pretrained_model_name_or_path": self.args.tokenizer_dir}
        Encoder.tokenizer = build_tokenizer(cfg)

    def encode(self, line: str):
        line = line.strip()
        if not line:
            return {}, {}, 0
        record = json.loads(line)
        ids, lens = {}, {}
        tok = Encoder.tokenizer
        for key in self.args.json_keys:
            text = record.get(key, "")
            sentences = [s for s in text.split("\n") if s] if self.args.split_sentences else [text]
            doc, sizes = [], []
            for s in sentences:
                t = tok.encode(s, add_special_tokens=False)
                if t:
                    doc.extend(t)
                    sizes.append(len(t))
            if doc and self.args.append_eod:
                doc.append(getattr(tok, "eos_token_id", 0) or 0)
                sizes[-1] += 1
            ids[key], lens[key] = doc, sizes
        return ids, lens, len(line)


def process_partition(args, lines, prefix, vocab_size):
    enc = Encoder(args)
    builders = {k: IndexedDatasetBuilder(get_bin_path(f"{prefix}_{k}_document"), dtype=best_dtype(vocab_size)) for k in args.json_keys}
    if args.workers > 1:
        pool = multiprocessing.Pool(args.workers, initializer=enc.initializer)
        stream = pool.imap(enc.encode, lines, 32)
    else:
        enc.initializer()
        pool, stream = None, map(enc.encode, lines)
    t0, nbytes, ndocs = time.time(), 0, 0
    for ids, lens, n in stream:
        nbytes += n
        for key, doc in ids.items():
            if doc:
                builders[key].add_document(doc, lens[key])
                ndocs += 1
        if ndocs and ndocs % args.log_interval == 0:
            print(f"processed {ndocs} documents ({nbytes / 1e6 / max(time.time() - t0, 1e-6):.2f} MB/s)", flush=True)
    if pool is not None:
        pool.close()
        pool.join()
    for key, b in builders.items():
        b.finalize(get_idx_path(f"{prefix}_{key}_document"))
    return ndocs


def main(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("--input", required=True)
    p.add_argument("--output-prefix", required=True)
    p.add_argument("--json-keys", nargs="+", default=["text"])
    p.add_argument("--tokenizer-type", default="ByteTokenizer")
    p.add_argument("--tokenizer-dir", default=None, help="directory with tokenizer files (AutoTokenizer)")
    p.add_argument("--vocab-size", type=int, default=None)
    p.add_argument("--split-sentences", action="store_true")
    p.add_argument("--append-eod", action="store_true")
    p.add_argument("--workers", type=int, default=1)
    p.add_argument("--partitions", type=int, default=1)
    p.add_argument("--log-interval", type=int, default=10000)
    args = p.parse_args(argv)
    os.makedirs(os.path.dirname(os.path.abspath(args.output_prefix)) or ".", exist_ok=True)
    with open(args.input, encoding="utf-8") as f:
        lines = f.readlines()
    from mindformers_b200.models import build_tokenizer
    vocab = args.vocab_size or len(build_tokenizer({"type": args.tokenizer_type}) if not args.tokenizer_dir else
                                   build_tokenizer({"type": "AutoTokenizer", "pretrained_model_name_or_path": args.tokenizer_dir}))
    parts = max(1, args.partitions)
    bounds = np.linspace(0, len(lines), parts + 1).astype(int)
    prefixes, total = [], 0
    for i in range(parts):
        prefix = args.output_prefix if parts == 1 else f"{args.output_prefix}_part{i}"
        total += process_partition(args, lines[bounds[i]:bounds[i + 1]], prefix, vocab)
        prefixes.append(prefix)
    if parts > 1:
        for key in args.json_keys:
            final = f"{args.output_prefix}_{key}_document"
            b = IndexedDatasetBuilder(get_bin_path(final), dtype=best_dtype(vocab))
            for pre in prefixes:
                b.add_index(f"{pre}_{key}_document")
            b.finalize(get_idx_path(final))
            for pre in prefixes:
                os.remove(get_bin_path(f"{pre}_{key}_document"))
                os.remove(get_idx_path(f"{pre}_{key}_document"))
    print(f"wrote {total} documents to {args.output_prefix}_<key>_document.bin/.idx")
    return total


if __name__ == "__main__":
    main()
