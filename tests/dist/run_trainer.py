"""Worker (gloo on CPU): runs ``Trainer(args=<config json>).train()`` on every rank of a torchrun job and lets rank 0
write the loss history to ``--out``. The parallel layout comes from the configuration, as with ``run_mindformer.py``."""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", required=True, help="JSON file with the full configuration")
    ap.add_argument("--out", required=True)
    args = ap.parse_args()
    with open(args.config) as f:
        cfg = json.load(f)
    import torch
    torch.set_num_threads(1)
    from mindformers_b200.trainer import Trainer
    t = Trainer(args=cfg)
    t.train()
    import torch.distributed as dist
    rank = dist.get_rank() if dist.is_initialized() else 0
    if rank == 0:
        with open(args.out, "w") as f:
            json.dump({"losses": t.trainer.loss_history}, f)
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
