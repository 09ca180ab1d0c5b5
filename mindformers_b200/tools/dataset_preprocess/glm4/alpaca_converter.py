"""Alpaca records → GLM-4 chat messages: ``{"messages": [{"role": "user", …}, {"role": "assistant", …}]}`` per line
(reference ``tools/dataset_preprocess/glm4/alpaca_converter.py``)."""
from __future__ import annotations

import argparse
import json


def convert(records):
    for r in records:
        user = r["instruction"] + (("\n" + r["input"]) if r.get("input") else "")
        yield {"messages": [{"role": "user", "content": user}, {"role": "assistant", "content": r["output"]}]}


def main(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("--data_path", default="alpaca_data.json")
    p.add_argument("--output_path", default="alpaca_glm4_data.jsonl")
    args = p.parse_args(argv)
    with open(args.data_path, "r", encoding="utf-8") as f:
        records = json.load(f)
    with open(args.output_path, "w", encoding="utf-8") as f:
        for row in convert(records):
            f.write(json.dumps(row, ensure_ascii=False) + "\n")
    print(f"wrote {len(records)} conversations to {args.output_path}")


if __name__ == "__main__":
    main()
