"""WikiText (raw ``.tokens`` file, or JSON lines with a text key) → indexed dataset (``.bin`` + ``.idx``) of fixed-length
training samples (reference ``research/deepseek3/wikitext_to_bin.py``).

Every sample is ``seq_length + 1`` tokens, so that the shifted labels come from the same sample. ``--pad-or-stitch
stitch`` concatenates all articles (each followed by the end-of-document token) into one stream and cuts it into
samples; ``pad`` makes one sample per article, truncated or padded with the pad token."""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from mindformers_b200.dataset.dataloaders import wikitext_reader  # noqa: E402
from mindformers_b200.dataset.indexed_dataset import IndexedDatasetBuilder, best_dtype, get_bin_path, get_idx_path  # noqa: E402


def build_parser():
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--input", required=True, help="wiki.train.tokens, or a .json / .jsonl file")
    p.add_argument("--json-keys", nargs="+", default=["text"])
    p.add_argument("--tokenizer-type", default="LlamaTokenizerFast")
    p.add_argument("--tokenizer-dir", default=None, help="directory with the tokenizer files (AutoTokenizer)")
    p.add_argument("--vocab-file", default=None)
    p.add_argument("--merges-file", default=None)
    p.add_argument("--tokenizer-file", default=None)
    p.add_argument("--vocab-size", type=int, default=None)
    p.add_argument("--append-eod", action="store_true", help="pad mode: end every article with the end-of-document token")
    p.add_argument("--output-prefix", required=True)
    p.add_argument("--seq-length", type=int, default=4096)
    p.add_argument("--pad-or-stitch", default="stitch", choices=["pad", "stitch"])
    p.add_argument("--workers", type=int, default=1)
    p.add_argument("--log-interval", type=int, default=1000)
    return p


def build_tokenizer(args):
    from mindformers_b200.models import build_tokenizer as _build
    if args.tokenizer_dir:
        return _build({"type": "AutoTokenizer", "pretrained_model_name_or_path": args.tokenizer_dir})
    cfg = {"type": args.tokenizer_type}
    for key in ("vocab_file", "merges_file", "tokenizer_file"):
        if getattr(args, key):
            cfg[key] = getattr(args, key)
    return _build(cfg)


def read_texts(path: str, keys):
    if path.endswith((".json", ".jsonl")):
        with open(path, encoding="utf-8") as f:
            head = f.read(1)
            f.seek(0)
            records = json.load(f) if head == "[" else [json.loads(line) for line in f if line.strip()]
        return ["\n".join(str(r[k]) for k in keys if r.get(k)) for r in records]
    return [r["text"] for r in wikitext_reader(path)]


def make_samples(docs, seq_length: int, mode: str, eod: int, pad: int, append_eod: bool):
    """``docs``: token-id lists. Yields samples of exactly ``seq_length + 1`` ids."""
    width = seq_length + 1
    if mode == "stitch":
        stream = []
        for d in docs:
            stream.extend(d)
            stream.append(eod)
            while len(stream) >= width:
                yield stream[:width]
                stream = stream[width:]
        return                                   # the tail shorter than a sample is dropped
    for d in docs:
        d = list(d) + ([eod] if append_eod else [])
        d = d[:width]
        yield d + [pad] * (width - len(d))


def main(argv=None):
    args = build_parser().parse_args(argv)
    tok = build_tokenizer(args)
    eod = tok.eos_token_id if getattr(tok, "eos_token_id", None) is not None else 0
    pad = tok.pad_token_id if getattr(tok, "pad_token_id", None) is not None else eod
    texts = read_texts(args.input, args.json_keys)
    if args.workers > 1:
        import multiprocessing
        with multiprocessing.Pool(args.workers) as pool:
            docs = pool.map(_Encode(tok), texts, 16)
    else:
        docs = [tok.encode(t, add_special_tokens=False) for t in texts]
    docs = [list(d) for d in docs if len(d)]
    vocab = args.vocab_size or getattr(tok, "vocab_size", None) or (max(max(d) for d in docs) + 1)
    os.makedirs(os.path.dirname(os.path.abspath(args.output_prefix)) or ".", exist_ok=True)
    prefix = f"{args.output_prefix}_text_document"
    builder = IndexedDatasetBuilder(get_bin_path(prefix), dtype=best_dtype(max(vocab, eod + 1, pad + 1)))
    n = 0
    for sample in make_samples(docs, args.seq_length, args.pad_or_stitch, eod, pad, args.append_eod):
        builder.add_document(sample, [len(sample)])
        n += 1
        if n % args.log_interval == 0:
            print(f"wrote {n} samples", flush=True)
    builder.finalize(get_idx_path(prefix))
    print(f"{n} samples of {args.seq_length + 1} tokens from {len(docs)} articles -> {prefix}.bin / .idx")
    return prefix, n


class _Encode:
    def __init__(self, tok):
        self.tok = tok

    def __call__(self, text):
        return self.tok.encode(text, add_special_tokens=False)


if __name__ == "__main__":
    main()
