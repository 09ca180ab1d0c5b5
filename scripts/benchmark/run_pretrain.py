#!/usr/bin/env python
"""Pre-training / fine-tuning from one command (reference ``scripts/benchmark/run_pretrain.py:61-400`` ``ModelPretrain``):

    python scripts/benchmark/run_pretrain.py --model_name_or_dir llama3_1_8b --pretrain_data wiki.train.tokens
    python scripts/benchmark/run_pretrain.py --model_name_or_dir /path/to/model_dir --pretrain_data alpaca_data.json \\
        --input_args data_seq_len=2048 model_num_layers=4 data_batch_size=2

``--model_name_or_dir`` is resolved by ``BaseInitModel`` (a directory with one YAML and optional weights, a shipped
configuration name or a preset). ``--pretrain_data`` may be: nothing (synthetic tokens of the configured shape: a
throughput run), a ``.bin`` / ``.idx`` prefix or ``.jsonl`` / ``.npy`` token file (used as it is), a WikiText style text
file (tokenised, packed into samples of ``seq_length + 1`` and written as an indexed dataset) or an Alpaca style
``.json`` file (converted to conversations, rendered and tokenised with labels only on the replies). The tokenizer is
the model directory's, else a byte tokenizer. Weights in the model directory (or ``load_checkpoint=...``) turn the run
into fine-tuning. Prints one JSON line: steps, tokens/s and ms/step of the second half of the run, final loss."""
import argparse
import json
import os
import sys
import tempfile

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from base_init_model import BaseInitModel  # noqa: E402


def convert_type(text: str):
    """``"4"`` → 4, ``"0.5"`` → 0.5, ``"true"`` → True, ``"none"`` → None, anything else stays a string."""
    low = text.lower()
    if low in ("true", "false"):
        return low == "true"
    if low in ("none", "null"):
        return None
    for cast in (int, float):
        try:
            return cast(text)
        except ValueError:
            pass
    return text


def build_args(pairs):
    """``["a=1", "b=x"]`` → ``{"a": 1, "b": "x"}``."""
    out = {}
    for item in pairs or []:
        if "=" not in item:
            raise ValueError(f"--input_args takes key=value pairs, got {item!r}")
        k, v = item.split("=", 1)
        out[k.strip()] = convert_type(v.strip())
    return out


class ModelPretrain(BaseInitModel):
    def __init__(self, model_name_or_dir: str = "llama3_1_8b", input_args=None):
        super().__init__(model_name_or_dir, input_args, build_model=False)   # the trainer builds the network itself

    # ---- data ------------------------------------------------------------------------------------------------------
    def process_tokenizer(self):
        from mindformers_b200.models import AutoTokenizer, ByteTokenizer
        if self.model_path:
            try:
                return AutoTokenizer.from_pretrained(self.model_path)
            except Exception as exc:   # noqa: BLE001
                self.logger.warning("no tokenizer under %s (%s): using the byte tokenizer", self.model_path, exc)
        return ByteTokenizer()

    @staticmethod
    def generate_dataset_name(dataset_type: str, seq_length: int) -> str:
        return f"{dataset_type}{seq_length}"

    def generate_pretrain_data(self, pretrain_data, temp_dir: str):
        """Returns the ``train_dataset.data_loader`` section for ``pretrain_data`` (see the module docstring)."""
        mc = self.config["model"]["model_config"]
        seq = int(mc.get("seq_length") or 2048)
        if not pretrain_data:
            return {"type": "MockDataLoader", "seq_length": seq, "num_samples": 8192}
        if os.path.exists(pretrain_data + ".bin") and os.path.exists(pretrain_data + ".idx"):
            return {"type": "IndexedDataLoader", "path_prefix": pretrain_data, "seq_length": seq}
        if not os.path.isfile(pretrain_data):
            raise ValueError(f"{pretrain_data} does not exist or is not a file")
        name = os.path.basename(pretrain_data).lower()
        ext = os.path.splitext(name)[-1]
        if ext in (".jsonl", ".npy"):
            return {"type": "CommonDataLoader", "path": pretrain_data, "seq_length": seq}
        if ext == ".json" or "alpaca" in name:
            return self._process_alpaca_file(pretrain_data, temp_dir, seq)
        return self._process_wiki_file(pretrain_data, temp_dir, seq)

    def _process_wiki_file(self, path: str, temp_dir: str, seq: int):
        import numpy as np
        from mindformers_b200.dataset.indexed_dataset import IndexedDatasetBuilder
        from mindformers_b200.tools.dataset_preprocess.llama.llama_preprocess import tokenize_wiki
        tok = self.process_tokenizer()
        samples = tokenize_wiki(tok, [path], seq)
        if not samples:
            raise ValueError(f"{path} holds fewer than {seq + 1} tokens: nothing to train on")
        prefix = os.path.join(temp_dir, self.generate_dataset_name("wiki", seq))
        builder = IndexedDatasetBuilder(prefix + ".bin", dtype=np.int32)
        for s in samples:
            builder.add_document(np.asarray(s, dtype=np.int32), [len(s)])
        builder.finalize(prefix + ".idx")
        self.logger.info("%d samples of %d tokens from %s -> %s", len(samples), seq + 1, path, prefix)
        self._check_vocab(max(max(s) for s in samples))
        return {"type": "IndexedDataLoader", "path_prefix": prefix, "seq_length": seq}

    def _process_alpaca_file(self, path: str, temp_dir: str, seq: int):
        from mindformers_b200.tools.dataset_preprocess.llama import alpaca_converter
        from mindformers_b200.tools.dataset_preprocess.llama.llama_preprocess import tokenize_qa
        tok = self.process_tokenizer()
        conv = os.path.join(temp_dir, "alpaca-data-conversation.json")
        alpaca_converter.main(["--data_path", path, "--output_path", conv])
        rows = tokenize_qa(tok, conv, seq)
        out = os.path.join(temp_dir, self.generate_dataset_name("alpaca", seq) + ".jsonl")
        with open(out, "w", encoding="utf-8") as f:
            for r in rows:
                f.write(json.dumps(r) + "\n")
        self._check_vocab(max(max(r["input_ids"]) for r in rows))
        return {"type": "CommonDataLoader", "path": out, "seq_length": seq, "input_columns": ["input_ids", "labels"]}

    def _check_vocab(self, top_id: int):
        mc = self.config["model"]["model_config"]
        vocab = int(mc.get("vocab_size") or mc.get("padded_vocab_size") or 0)
        if vocab and top_id >= vocab:
            raise ValueError(f"token id {top_id} does not fit the model's vocabulary of {vocab}: give a model directory "
                             "with its tokenizer, or a configuration whose vocab_size covers the tokenizer")

    # ---- run -------------------------------------------------------------------------------------------------------
    def train(self, pretrain_data=None, steps=None, output_dir=None):
        from mindformers_b200.core.callback import MFLossMonitor
        from mindformers_b200.trainer import Trainer
        cfg = self.config
        with tempfile.TemporaryDirectory(prefix="mfb_pretrain_") as tmp:
            cfg["train_dataset"]["data_loader"] = self.generate_pretrain_data(pretrain_data, tmp)
            cfg["run_mode"] = "finetune" if self.finetune else "train"
            if steps:
                cfg.set_value("runner_config.stop_step", int(steps))
            if output_dir:
                cfg["output_dir"] = output_dir
            if not any((c or {}).get("type") == "MFLossMonitor" for c in cfg.get("callbacks") or []):
                cfg["callbacks"] = list(cfg.get("callbacks") or []) + [{"type": "MFLossMonitor"}]
            self.logger.info("starting a %s run of %s", cfg["run_mode"], self.model_name)
            trainer = Trainer(cfg)
            trainer.train()
        mon = next(c for c in trainer.trainer.callbacks if isinstance(c, MFLossMonitor))
        tail = mon.history[len(mon.history) // 2:] or mon.history
        return {"model": self.model_name, "mode": cfg["run_mode"], "steps": len(mon.history),
                "tokens_per_s": sum(r["tokens_per_s"] for r in tail) / len(tail),
                "ms_per_step": sum(r["step_ms"] for r in tail) / len(tail), "final_loss": mon.history[-1]["loss"]}


def main(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("--model_name_or_dir", default=None)
    p.add_argument("--config", default=None, help="a YAML file (its directory is not searched for weights)")
    p.add_argument("--pretrain_data", default=None)
    p.add_argument("--steps", type=int, default=None)
    p.add_argument("--output_dir", default="./output_benchmark")
    p.add_argument("--input_args", nargs="*", default=[], help="key=value overrides, see base_init_model.py")
    args = p.parse_args(argv)
    overrides = build_args(args.input_args)
    if args.config:
        # a bare YAML: stage it in a directory of its own so that BaseInitModel treats it as a model directory
        import shutil
        stage = tempfile.mkdtemp(prefix="mfb_cfg_")
        shutil.copy(os.path.abspath(args.config), os.path.join(stage, os.path.basename(args.config)))
        target = stage
    else:
        target = args.model_name_or_dir or "tiny_llama"
    runner = ModelPretrain(target, overrides)
    result = runner.train(args.pretrain_data, args.steps, args.output_dir)
    print(json.dumps(result))
    return result


if __name__ == "__main__":
    main()
