"""Raw text / conversation files → fixed-length token samples for Llama pre-training and fine-tuning.

    python -m mindformers_b200.tools.dataset_preprocess.llama.llama_preprocess --dataset_type wiki \\
        --input_glob wiki.train.tokens --model_file tokenizer.model --seq_length 2048 --output_file out/wiki2048

``wiki``: the text is cleaned (WikiText spacing), tokenised, documents are joined with ``eos`` and cut into samples of
``seq_length + 1`` tokens (``input_ids``). ``qa``: conversation records (see ``alpaca_converter``) are rendered with the
Vicuna template; labels are ``-100`` except on assistant replies. The output is ``<output_file>.jsonl`` (one sample
per line) plus, for ``wiki``, the Megatron ``.bin/.idx`` pair that ``IndexedDataLoader`` reads — the reference wrote
MindRecord files here (``tools/dataset_preprocess/llama/llama_preprocess.py:194-275``).
"""
from __future__ import annotations

import argparse
import glob
import json
import os
from typing import Dict, Iterable, List

import numpy as np

from ....dataset.dataloaders import wikitext_reader
from .conversation import get_default_conv_template

IGNORE = -100


def tokenize_wiki(tokenizer, files: Iterable[str], seq_length: int, repeat: int = 1) -> List[List[int]]:
    stream: List[int] = []
    for path in files:
        for row in wikitext_reader(path):
            stream += list(tokenizer.encode(row["text"], add_special_tokens=False)) + [tokenizer.eos_token_id]
    stream = stream * repeat
    width = seq_length + 1
    return [stream[i:i + width] for i in range(0, len(stream) - width + 1, width)]


def tokenize_qa(tokenizer, path: str, seq_length: int) -> List[Dict[str, List[int]]]:
    """Labels follow the template boundaries: everything up to and including ``ASSISTANT:`` of a round is ignored."""
    with open(path, "r", encoding="utf-8") as f:
        records = json.load(f)
    samples = []
    for rec in records:
        conv = get_default_conv_template()
        roles = {"human": conv.roles[0], "gpt": conv.roles[1]}
        ids: List[int] = [tokenizer.bos_token_id] if tokenizer.bos_token_id is not None else []
        labels: List[int] = [IGNORE] * len(ids)
        head = list(tokenizer.encode(conv.system + conv.sep, add_special_tokens=False))
        ids += head
        labels += [IGNORE] * len(head)
        for turn in rec["conversations"]:
            role = roles.get(turn["from"], turn["from"])
            if turn["from"] == "gpt":
                q = list(tokenizer.encode(f"{role}: ", add_special_tokens=False))
                a = list(tokenizer.encode(turn["value"], add_special_tokens=False)) + [tokenizer.eos_token_id]
                ids += q + a
                labels += [IGNORE] * len(q) + a
            else:
                q = list(tokenizer.encode(f"{role}: {turn['value']}{conv.sep}", add_special_tokens=False))
                ids += q
                labels += [IGNORE] * len(q)
        width = seq_length + 1
        pad = tokenizer.pad_token_id if tokenizer.pad_token_id is not None else 0
        ids, labels = ids[:width], labels[:width]
        gap = width - len(ids)
        samples.append({"input_ids": ids + [pad] * gap, "labels": labels + [IGNORE] * gap})
    return samples


def main(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("--dataset_type", default="wiki", choices=["wiki", "qa"])
    p.add_argument("--input_glob", required=True)
    p.add_argument("--output_file", default="./dataset/wiki2048/wiki2048")
    p.add_argument("--tokenizer", default="llama")
    p.add_argument("--model_file", required=True, help="tokenizer file or directory")
    p.add_argument("--repeat", type=int, default=1)
    p.add_argument("--seq_length", type=int, default=2048)
    args = p.parse_args(argv)
    from ....models import AutoTokenizer
    tok = AutoTokenizer.from_pretrained(args.model_file)
    os.makedirs(os.path.dirname(os.path.abspath(args.output_file)), exist_ok=True)
    files = sorted(glob.glob(args.input_glob))
    if not files:
        raise FileNotFoundError(f"no file matches {args.input_glob}")
    if args.dataset_type == "wiki":
        samples = tokenize_wiki(tok, files, args.seq_length, args.repeat)
        from ....dataset.indexed_dataset import IndexedDatasetBuilder
        builder = IndexedDatasetBuilder(args.output_file + ".bin", dtype=np.int32)
        for s in samples:
            builder.add_document(np.asarray(s, dtype=np.int32), [len(s)])
        builder.finalize(args.output_file + ".idx")
        rows = [{"input_ids": s} for s in samples]
    else:
        rows = [r for f in files for r in tokenize_qa(tok, f, args.seq_length)]
    with open(args.output_file + ".jsonl", "w", encoding="utf-8") as f:
        for r in rows:
            f.write(json.dumps(r) + "\n")
    print(f"wrote {len(rows)} samples of {args.seq_length + 1} tokens to {args.output_file}.jsonl")
    return len(rows)


if __name__ == "__main__":
    main()
