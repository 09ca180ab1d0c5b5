"""One serving worker per GPU: builds a ``ModelRunner`` and answers line-delimited JSON requests on stdin (rank 0) —
``{"op": "forward", ...}`` / ``{"op": "swap", ...}`` / ``{"op": "stop"}`` — broadcasting each request to the other
ranks. A serving engine normally embeds ``ModelRunner`` directly; this loop is the reference wiring and a smoke test."""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

from .model_runner import ModelRunner


def main(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("--model_dir", required=True)
    p.add_argument("--gpu_mem_gb", type=float, default=40)
    p.add_argument("--cpu_mem_gb", type=float, default=8)
    p.add_argument("--block_size", type=int, default=128)
    a = p.parse_args(argv)
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    runner = ModelRunner(a.model_dir, a.gpu_mem_gb, a.cpu_mem_gb, a.block_size, rank_id=rank, world_size=world)
    while True:
        box = [None]
        if rank == 0:
            line = sys.stdin.readline()
            box[0] = json.loads(line) if line.strip() else {"op": "stop"}
        if world > 1:
            dist.broadcast_object_list(box, src=0)
        req = box[0]
        if req["op"] == "stop":
            break
        if req["op"] == "swap":
            runner.swap(req["block_tables"], bool(req["swap_out"]))
            continue
        logits = runner.forward(np.asarray(req["input_ids"]), req["valid_length_each_example"], np.asarray(req["block_tables"]),
                                np.asarray(req["slot_mapping"]), prefill=bool(req.get("prefill", True)))
        if rank == 0:
            print(json.dumps({"next_tokens": logits.argmax(-1).tolist()}), flush=True)


if __name__ == "__main__":
    main()
