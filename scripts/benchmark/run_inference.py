#!/usr/bin/env python
"""Offline generation benchmark from a model directory (``scripts/benchmark/run_inference.py:41 ModelPredict``):

    python scripts/benchmark/run_inference.py --model_dir /path/to/model --prompts "hello" "hi" --max_new_tokens 128

Reports tokens/s as the reference does (generated tokens / total wall time, ``generation/text_generator.py:1108-1111``)
plus time to first token."""
import argparse
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)


def main(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("--model_dir", default=None)
    p.add_argument("--preset", default=None, help="random-init model of a named preset instead of a directory")
    p.add_argument("--prompts", nargs="*", default=["Hello, my name is"])
    p.add_argument("--prompt_tokens", type=int, default=0, help="use random prompts of this many tokens instead")
    p.add_argument("--batch_size", type=int, default=1)
    p.add_argument("--max_new_tokens", type=int, default=64)
    p.add_argument("--layers", type=int, default=None)
    args = p.parse_args(argv)
    import torch
    from mindformers_b200.models import AutoModel, AutoTokenizer, ByteTokenizer
    from mindformers_b200.models.presets import get_preset
    if args.model_dir:
        model = AutoModel.from_pretrained(args.model_dir)
        try:
            tok = AutoTokenizer.from_pretrained(args.model_dir)
        except Exception:
            tok = ByteTokenizer()
    else:
        cfg = get_preset(args.preset or "tiny_llama")
        if args.layers:
            cfg["num_hidden_layers"] = args.layers
        model = AutoModel.from_config(cfg)
        tok = ByteTokenizer()
    model.eval()
    if args.prompt_tokens:
        g = torch.Generator().manual_seed(0)
        prompts = torch.randint(3, model.config.vocab_size, (args.batch_size, args.prompt_tokens), generator=g).tolist()
    else:
        prompts = [tok.encode(t) for t in args.prompts]
    model.generate(prompts[:1], max_new_tokens=2)                     # warm-up
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    t0 = time.perf_counter()
    first = model.generate(prompts, max_new_tokens=1)
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    ttft = time.perf_counter() - t0
    t0 = time.perf_counter()
    out = model.generate(prompts, max_new_tokens=args.max_new_tokens)
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    new = sum(len(o) - len(pr) for o, pr in zip(out, prompts))
    print(json.dumps({"batch": len(prompts), "new_tokens": new, "seconds": dt, "tokens_per_s": new / dt, "ttft_s": ttft}))
    if not args.prompt_tokens:
        for o in out[:2]:
            print(tok.decode(o))
    del first


if __name__ == "__main__":
    main()
