#!/usr/bin/env python
"""Pre-training throughput from a YAML or a preset (``scripts/benchmark/run_pretrain.py:61 ModelPretrain``):

    python scripts/benchmark/run_pretrain.py --config configs/general/run_general_task.yaml --steps 10

Runs ``Trainer.train`` for ``--steps`` steps on synthetic tokens and prints the mean tokens/s of the last half."""
import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)


def main(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("--config", required=True)
    p.add_argument("--steps", type=int, default=10)
    p.add_argument("--output_dir", default="./output_benchmark")
    args = p.parse_args(argv)
    from mindformers_b200.core.callback import MFLossMonitor
    from mindformers_b200.tools.register.config import MindFormerConfig
    from mindformers_b200.trainer import Trainer
    cfg = MindFormerConfig(os.path.abspath(args.config))
    cfg.set_value("runner_config.stop_step", args.steps)
    cfg["output_dir"] = args.output_dir
    cfg["callbacks"] = [{"type": "MFLossMonitor"}]
    t = Trainer(cfg)
    t.train()
    mon = next(c for c in t.trainer.callbacks if isinstance(c, MFLossMonitor))
    tail = mon.history[len(mon.history) // 2:]
    print(json.dumps({"steps": len(mon.history), "tokens_per_s": sum(r["tokens_per_s"] for r in tail) / len(tail),
                      "ms_per_step": sum(r["step_ms"] for r in tail) / len(tail), "final_loss": mon.history[-1]["loss"]}))


if __name__ == "__main__":
    main()
