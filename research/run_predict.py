"""Shared body of the per-model predict scripts (``research/qwen2_5/run_qwen2_5.py``, ``research/deepseek3/
run_predict_deepseek.py``, ``research/telechat2/run_telechat_predict.py`` of the reference): read a predict YAML, apply
the command-line overrides those scripts take, build the trainer and generate for the given prompts.

The reference's scripts differ in flag spelling only (``--config`` / ``--yaml_file``, ``--load_checkpoint`` /
``--checkpoint_path``, ``--vocab_file`` / ``--vocab_file_path``, ``--predict_length`` / ``--max_length``); both
spellings are accepted here."""
from __future__ import annotations

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def str2bool(v):
    if isinstance(v, bool):
        return v
    if str(v).lower() in ("true", "1", "yes", "y"):
        return True
    if str(v).lower() in ("false", "0", "no", "n"):
        return False
    raise argparse.ArgumentTypeError(f"expected a boolean, got {v!r}")


def build_parser(default_config=None, default_prompt="") -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--task", default="text_generation")
    p.add_argument("--config", "--yaml_file", dest="config", default=default_config, help="predict YAML")
    p.add_argument("--run_mode", default="predict")
    p.add_argument("--load_checkpoint", "--checkpoint_path", dest="load_checkpoint", default=None)
    p.add_argument("--auto_trans_ckpt", default=None, type=str2bool)
    p.add_argument("--src_strategy_path_or_dir", default=None)
    p.add_argument("--vocab_file", "--vocab_file_path", dest="vocab_file", default=None)
    p.add_argument("--merges_file", default=None)
    p.add_argument("--tokenizer_file", default=None)
    p.add_argument("--predict_data", "--input", dest="predict_data", default=default_prompt, nargs="*",
                   help="prompt text(s), or a file with one prompt per line")
    p.add_argument("--seq_length", default=None, type=int)
    p.add_argument("--predict_length", "--max_length", dest="max_length", default=None, type=int)
    p.add_argument("--max_new_tokens", default=None, type=int)
    p.add_argument("--use_parallel", default=None, type=str2bool)
    p.add_argument("--device_id", default=None, type=int)
    p.add_argument("--use_past", default=None, type=str2bool)
    p.add_argument("--do_sample", default=None, type=str2bool)
    p.add_argument("--top_k", default=None, type=int)
    p.add_argument("--top_p", default=None, type=float)
    p.add_argument("--repetition_penalty", default=None, type=float)
    p.add_argument("--batch_size", default=None, type=int)
    return p


def apply_overrides(config, args):
    """Command-line values → the places of the configuration that the trainer reads."""
    model_cfg = config.model.model_config
    if args.seq_length is not None:
        model_cfg.seq_length = args.seq_length
    if args.use_past is not None:
        model_cfg.use_past = args.use_past
    if args.use_parallel is not None:
        config.use_parallel = args.use_parallel
    if args.device_id is not None and config.get("context") is not None:
        config.context.device_id = args.device_id
    if args.load_checkpoint:
        config.load_checkpoint = args.load_checkpoint
    if args.auto_trans_ckpt is not None:
        config.auto_trans_ckpt = args.auto_trans_ckpt
    if args.src_strategy_path_or_dir:
        config.src_strategy_path_or_dir = args.src_strategy_path_or_dir
    if args.batch_size is not None:
        config.predict_batch_size = args.batch_size
    tok = (config.get("processor") or {}).get("tokenizer")
    if tok is not None:
        for key in ("vocab_file", "merges_file", "tokenizer_file"):
            if getattr(args, key):
                tok[key] = getattr(args, key)
    gen = config.get("generation") or config.get("generation_config")
    if gen is None:
        config["generation"] = gen = type(config)()
    for key in ("max_length", "max_new_tokens", "do_sample", "top_k", "top_p", "repetition_penalty"):
        v = getattr(args, key)
        if v is not None:
            gen[key] = v
            model_cfg[key] = v
    config.run_mode = args.run_mode
    return config


def prompts_of(values):
    if isinstance(values, str):
        values = [values]
    values = [v for v in values if v != ""]
    if len(values) == 1 and os.path.isfile(values[0]):
        with open(values[0], encoding="utf-8") as f:
            return [line.rstrip("\n") for line in f if line.strip()]
    return values


def main(argv=None, default_config=None, default_prompt="", wrap_prompt=None):
    """``wrap_prompt``: a function prompt → text that applies the model's chat format (the reference scripts hard-code it)."""
    args = build_parser(default_config, default_prompt).parse_args(argv)
    if not args.config:
        raise SystemExit("--config (a predict YAML) is required")
    from mindformers_b200.core.context import build_context
    from mindformers_b200.tools.register import MindFormerConfig
    from mindformers_b200.trainer import Trainer
    config = apply_overrides(MindFormerConfig(os.path.abspath(args.config)), args)
    prompts = prompts_of(args.predict_data)
    if not prompts:
        raise SystemExit("no prompt given (--predict_data)")
    if wrap_prompt is not None:
        prompts = [wrap_prompt(p) for p in prompts]
    build_context(config)
    trainer = Trainer(config)
    result = trainer.predict(predict_checkpoint=config.get("load_checkpoint") or None, input_data=prompts if len(prompts) > 1 else prompts[0],
                             batch_size=config.get("predict_batch_size"))
    rows = result
    if isinstance(result, dict):
        rows = next((v for v in result.values() if isinstance(v, (list, tuple))), [result])
    for row in rows or []:
        print(row)
    return result


if __name__ == "__main__":
    main()
