"""GLM-4 chat messages (jsonl) → ``input_ids`` / ``labels`` samples of ``seq_length`` tokens (jsonl).

    python -m mindformers_b200.tools.dataset_preprocess.glm4.glm4_preprocess --input_glob data.jsonl \\
        --vocab_file tokenizer.model --seq_length 8192 --output_file out/glm4

Turns are rendered with the tokenizer's role tokens (``[gMASK] <sop> <|user|>\\n…<|assistant|>\\n…``); only assistant
turns carry labels (reference ``tools/dataset_preprocess/glm4/glm4_preprocess.py``).
"""
from __future__ import annotations

import argparse
import glob
import json
import os

IGNORE = -100


def encode_messages(tokenizer, messages, seq_length: int):
    ids = list(tokenizer.get_prefix_tokens())
    labels = [IGNORE] * len(ids)
    for m in messages:
        part = list(tokenizer.build_single_message(m["role"], m.get("metadata", ""), m["content"]))
        ids += part
        labels += part if m["role"] == "assistant" else [IGNORE] * len(part)
    ids.append(tokenizer.eos_token_id)
    labels.append(tokenizer.eos_token_id if messages and messages[-1]["role"] == "assistant" else IGNORE)
    ids, labels = ids[:seq_length], labels[:seq_length]
    gap = seq_length - len(ids)
    pad = tokenizer.pad_token_id if tokenizer.pad_token_id is not None else 0
    return {"input_ids": ids + [pad] * gap, "labels": labels + [IGNORE] * gap}


def main(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("--input_glob", required=True)
    p.add_argument("--vocab_file", required=True)
    p.add_argument("--seq_length", type=int, default=8192)
    p.add_argument("--output_file", default="./dataset/glm4")
    args = p.parse_args(argv)
    from ....models import ChatGLM4Tokenizer
    tok = ChatGLM4Tokenizer(args.vocab_file)
    os.makedirs(os.path.dirname(os.path.abspath(args.output_file)), exist_ok=True)
    n = 0
    with open(args.output_file + ".jsonl", "w", encoding="utf-8") as out:
        for path in sorted(glob.glob(args.input_glob)):
            with open(path, "r", encoding="utf-8") as f:
                for line in f:
                    if line.strip():
                        out.write(json.dumps(encode_messages(tok, json.loads(line)["messages"], args.seq_length)) + "\n")
                        n += 1
    print(f"wrote {n} samples to {args.output_file}.jsonl")
    return n


if __name__ == "__main__":
    main()
