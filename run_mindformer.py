#!/usr/bin/env python
"""Single command-line entry for train / finetune / eval / predict.

    python run_mindformer.py --config configs/llama3_1/pretrain_llama3_1_8b.yaml --run_mode train
    torchrun --nproc-per-node 8 --master-addr 127.0.0.1 run_mindformer.py --config X.yaml --use_parallel True

Precedence of settings (lowest first): YAML (``base_config`` parents, then the child) < the named flags below
< ``--options k=v`` < free ``--a.b.c=v`` overrides — the order of the reference's ``run_mindformer.py:238-338``.
``--register_path`` exports ``REGISTER_PATH`` so classes named by ``auto_register`` are found (:225-231).
"""
import argparse
import os
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from mindformers_b200.tools.register.config import ActionDict, MindFormerConfig, parse_value  # noqa: E402
from mindformers_b200.tools.utils import str2bool  # noqa: E402

# flag → (dotted configuration key, parser type)
NAMED_FLAGS = {
    "mode": ("context.mode", int), "device_id": ("context.device_id", int), "device_target": ("context.device_target", str),
    "run_mode": ("run_mode", str), "do_eval": ("do_eval", str2bool),
    "train_dataset_dir": ("train_dataset.data_loader.dataset_dir", str), "eval_dataset_dir": ("eval_dataset.data_loader.dataset_dir", str),
    "predict_batch_size": ("predict_batch_size", int), "adapter_id": ("adapter_id", str),
    "load_checkpoint": ("load_checkpoint", str), "src_strategy_path_or_dir": ("src_strategy_path_or_dir", str),
    "auto_trans_ckpt": ("auto_trans_ckpt", str2bool), "transform_process_num": ("transform_process_num", int),
    "only_save_strategy": ("only_save_strategy", str2bool), "resume_training": ("resume_training", parse_value),
    "strategy_load_checkpoint": ("parallel.strategy_ckpt_load_file", str), "remote_save_url": ("remote_save_url", str),
    "seed": ("seed", int), "use_parallel": ("use_parallel", str2bool), "profile": ("profile", str2bool),
    "epochs": ("runner_config.epochs", int), "batch_size": ("runner_config.batch_size", int),
    "gradient_accumulation_steps": ("runner_config.gradient_accumulation_steps", int),
    "sink_mode": ("runner_config.sink_mode", str2bool), "num_samples": ("train_dataset.data_loader.num_samples", int),
    "output_dir": ("output_dir", str), "do_sample": ("model.model_config.do_sample", str2bool),
    "modal_type": ("modal_type", str), "trust_remote_code": ("trust_remote_code", str2bool),
    "pretrained_model_dir": ("pretrained_model_dir", str), "save_file": ("save_file", str),
}


def build_parser():
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--config", required=True, help="YAML configuration file")
    for flag, (key, typ) in NAMED_FLAGS.items():
        p.add_argument(f"--{flag}", default=None, type=typ, help=f"overrides `{key}`")
    p.add_argument("--predict_data", default=None, nargs="+", help="prompt text(s) or a file with one prompt per line")
    p.add_argument("--register_path", default=None, help="directory searched for plug-in classes (auto_register)")
    p.add_argument("--options", nargs="+", action=ActionDict, default=None, help="k=v pairs merged into the configuration")
    return p


def load_config(argv=None) -> MindFormerConfig:
    parser = build_parser()
    args, rest = parser.parse_known_args(argv)
    if args.register_path:
        os.environ["REGISTER_PATH"] = os.path.abspath(args.register_path)
        if os.environ["REGISTER_PATH"] not in sys.path:
            sys.path.insert(0, os.environ["REGISTER_PATH"])
    config = MindFormerConfig(os.path.abspath(args.config))
    for flag, (key, _) in NAMED_FLAGS.items():
        v = getattr(args, flag)
        if v is not None:
            config.set_value(key, v)
    if args.predict_data is not None:
        data = args.predict_data
        config["input_data"] = data[0] if len(data) == 1 and os.path.isfile(data[0]) else (data if len(data) > 1 else data[0])
    if args.options:
        config.merge_from_dict(args.options)
    free = {}
    i = 0
    while i < len(rest):                      # free overrides: --a.b.c=v  or  --a.b.c v
        tok = rest[i]
        if not tok.startswith("--"):
            raise SystemExit(f"unrecognised argument {tok!r}")
        if "=" in tok:
            k, v = tok[2:].split("=", 1)
        else:
            if i + 1 >= len(rest):
                raise SystemExit(f"override {tok!r} needs a value")
            k, v = tok[2:], rest[i + 1]
            i += 1
        free[k] = parse_value(v)
        i += 1
    if free:
        config.merge_from_dict(free)
    return config


def main(config: MindFormerConfig):
    from mindformers_b200.core.context import build_context
    from mindformers_b200.tools.utils import set_output_path
    from mindformers_b200.trainer import Trainer
    set_output_path(config.get("output_dir"))
    if config.get("auto_register"):
        from mindformers_b200.tools.register.register import MindFormerRegister
        MindFormerRegister.auto_register(config["auto_register"])
    build_context(config)
    trainer = Trainer(config)
    mode = config.get("run_mode")
    if mode in ("train", "finetune"):
        return trainer.train() if mode == "train" else trainer.finetune()
    if mode == "eval":
        return trainer.evaluate(eval_checkpoint=config.get("load_checkpoint") or False)
    if mode == "predict":
        return trainer.predict(predict_checkpoint=config.get("load_checkpoint") or None, input_data=config.get("input_data"),
                               batch_size=config.get("predict_batch_size"))
    raise SystemExit(f"run_mode must be one of train/finetune/eval/predict, got {mode!r}")


if __name__ == "__main__":
    main(load_config())
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized():
        dist.destroy_process_group()
