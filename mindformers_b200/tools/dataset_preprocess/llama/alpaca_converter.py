"""Alpaca instruction records → multi-turn conversation records.

    python -m mindformers_b200.tools.dataset_preprocess.llama.alpaca_converter --data_path alpaca_data.json \\
        --output_path alpaca-data-conversation.json

Each ``{"instruction", "input", "output"}`` becomes ``{"id", "conversations": [{"from": "human", "value": prompt},
{"from": "gpt", "value": output}]}`` with the two Alpaca prompt templates (reference
``tools/dataset_preprocess/llama/alpaca_converter.py:48-112``).
"""
from __future__ import annotations

import argparse
import json

from ....dataset.dataloaders import ALPACA_NO_INPUT, ALPACA_WITH_INPUT


def convert(records):
    out = []
    for i, r in enumerate(records):
        tmpl = ALPACA_WITH_INPUT if r.get("input") else ALPACA_NO_INPUT
        prompt = tmpl.format(instruction=r["instruction"], input=r.get("input", ""))
        out.append({"id": str(i + 1), "conversations": [{"from": "human", "value": prompt},
                                                        {"from": "gpt", "value": r["output"]}]})
    return out


def main(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("--data_path", default="alpaca_data.json")
    p.add_argument("--output_path", default="alpaca-data-conversation.json")
    args = p.parse_args(argv)
    with open(args.data_path, "r", encoding="utf-8") as f:
        records = json.load(f)
    with open(args.output_path, "w", encoding="utf-8") as f:
        json.dump(convert(records), f, ensure_ascii=False, indent=2)
    print(f"wrote {len(records)} conversations to {args.output_path}")


if __name__ == "__main__":
    main()
