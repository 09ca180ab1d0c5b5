#!/usr/bin/env python
"""Common model set-up of the benchmark tools (reference ``scripts/benchmark/base_init_model.py:49-175``
``BaseInitModel``): resolve a model *directory* (one ``*.yaml`` plus optional weights) or a *name* (a shipped YAML under
``configs/`` or a preset of ``models/presets.py``) into a full configuration, apply the command-line overrides
(``data_batch_size``, ``data_seq_len``, ``model_num_layers``, ``data_parallel`` / ``model_parallel`` /
``pipeline_stage``, any key of ``model_config``, ``load_checkpoint``, ``auto_trans_ckpt``, ``src_strategy``), decide
between pre-training (no weights) and fine-tuning (weights found), and build the network (wrapped by the PEFT model
when the configuration has a ``pet_config``)."""
from __future__ import annotations

import copy
import glob
import os
import sys
from pathlib import Path
from typing import Optional

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WEIGHT_PATTERNS = ("*.safetensors", "*.ckpt", "*.pt")


def get_parallel_status():
    """(running under a multi-process launcher?, number of ranks)."""
    n = os.getenv("WORLD_SIZE") or os.getenv("MS_WORKER_NUM")
    return (True, int(n)) if n and int(n) > 1 else (False, 1)


def convert_path(src_path: str, save_path: str):
    """(real source path, where a link to it goes inside ``save_path``)."""
    src = os.path.realpath(src_path)
    return src, os.path.join(save_path, os.path.basename(src))


def _find_yaml_by_name(name: str) -> Optional[str]:
    """``llama3_1_8b`` → the shipped pre-training (else any) YAML whose file name carries that model name."""
    hits = sorted(glob.glob(os.path.join(ROOT, "configs", "**", f"*{name}*.yaml"), recursive=True))
    for prefer in ("pretrain", "finetune", "predict"):
        for h in hits:
            if os.path.basename(h).startswith(prefer):
                return h
    return hits[0] if hits else None


class BaseInitModel:
    """``BaseInitModel(model_name_or_dir, input_args)``: after construction ``config`` is the full configuration,
    ``network`` the model (on its device), ``model_name`` / ``model_path`` say what was resolved and
    ``finetune`` whether weights will be loaded."""

    def __init__(self, model_name_or_dir: str = "llama3_1_8b", input_args: Optional[dict] = None, build_model: bool = True):
        from mindformers_b200.models.presets import PRESETS, get_preset
        from mindformers_b200.tools.logger import logger
        from mindformers_b200.tools.register.config import MindFormerConfig
        self.logger = logger
        self.model_name_or_dir = model_name_or_dir
        self.input_args = dict(input_args or {})
        self.model_path: Optional[str] = None
        if Path(model_name_or_dir).is_dir():
            self.model_path = str(Path(model_name_or_dir).absolute())
            yamls = sorted(glob.glob(os.path.join(self.model_path, "*.yaml")))
            if not yamls:
                raise RuntimeError(f"no yaml file under {self.model_path}")
            self.config = MindFormerConfig(yamls[0])
            self.model_name = (self.config.get("trainer") or {}).get("model_name") or Path(self.model_path).name
            sys.path.append(self.model_path)           # model code shipped next to the yaml (auto_map / REGISTER_PATH)
        else:
            self.model_name = model_name_or_dir
            yaml_path = _find_yaml_by_name(model_name_or_dir)
            if yaml_path:
                self.config = MindFormerConfig(yaml_path)
            elif model_name_or_dir in PRESETS:
                base = MindFormerConfig(os.path.join(ROOT, "configs", "general", "run_general_task.yaml"))
                base["model"]["model_config"] = dict(get_preset(model_name_or_dir), architectures=["LlamaForCausalLM"])
                self.config = base
            else:
                raise ValueError(f"{model_name_or_dir!r} is neither a directory, a shipped configuration nor a preset "
                                 f"({sorted(PRESETS)})")
        self.custom_model = False
        self.use_pet_model = False
        self.finetune = False
        self.init_config()
        self.process_checkpoint()
        self.network = None
        if build_model:
            self.build_model()

    # ---- configuration -----------------------------------------------------------------------------------------
    def init_config(self):
        self.process_parallel_config()
        self.process_model_config()
        cfg, args = self.config, self.input_args
        ckpt = cfg.get("load_checkpoint") or ""
        auto = bool(cfg.get("use_parallel")) and os.path.isfile(ckpt)
        cfg["auto_trans_ckpt"] = args.get("auto_trans_ckpt", auto)
        mc = cfg["model"]["model_config"]
        if args.get("data_batch_size"):
            cfg["runner_config"]["batch_size"] = int(args["data_batch_size"])
        if args.get("data_seq_len"):
            seq = int(args["data_seq_len"])
            mc["seq_length"] = seq
            mc["max_position_embeddings"] = max(int(mc.get("max_position_embeddings") or 0), seq)
            loader = (cfg.get("train_dataset") or {}).get("data_loader")
            if isinstance(loader, dict) and "seq_length" in loader:
                loader["seq_length"] = seq
        if args.get("model_num_layers"):
            key = "num_hidden_layers" if "num_hidden_layers" in mc else "num_layers"
            mc[key] = int(args["model_num_layers"])
        if args.get("src_strategy"):
            cfg["src_strategy_path_or_dir"] = args["src_strategy"]

    def process_parallel_config(self):
        pc = self.config.get("parallel_config")
        if pc is None:
            return
        for key in ("data_parallel", "model_parallel", "pipeline_stage", "context_parallel", "expert_parallel",
                    "micro_batch_num", "use_seq_parallel"):
            if self.input_args.get(key) is not None:
                pc[key] = self.input_args[key]
        launched, n = get_parallel_status()
        if launched:
            self.config["use_parallel"] = True
            mp = int(pc.get("model_parallel", 1)) * int(pc.get("pipeline_stage", 1)) * int(pc.get("context_parallel", 1))
            if self.input_args.get("data_parallel") is None and n % mp == 0:
                pc["data_parallel"] = n // mp

    def process_model_config(self):
        mc = self.config["model"]["model_config"]
        mc["checkpoint_name_or_path"] = None           # weights come through load_checkpoint only
        if mc.get("pet_config"):
            self.use_pet_model = True
        for k, v in self.input_args.items():
            if k in mc and v is not None:
                self.custom_model = True
                mc[k] = v

    def process_checkpoint(self):
        """Pick the weights: an explicit ``load_checkpoint`` argument (``""`` / ``False`` = none: pre-training), else the
        configuration's, else the first weight file in the model directory. A file outside the model directory is
        linked into it, as the reference does, so that later runs find it there."""
        want = self.input_args.get("load_checkpoint", None)
        if want == "" or want is False:
            self.logger.warning("load_checkpoint is switched off: running [pretrain]")
            self.config["load_checkpoint"] = ""
            return
        if not want or not os.path.exists(str(want)):
            want = self.config.get("load_checkpoint") or None
        if want and os.path.exists(str(want)):
            if self.model_path and os.path.isfile(str(want)) and os.path.dirname(os.path.realpath(str(want))) != self.model_path:
                src, link = convert_path(str(want), self.model_path)
                try:
                    os.symlink(src, link)
                except OSError:
                    self.logger.warning("link %s -> %s exists already", src, link)
                want = link
            self.logger.info("checkpoint found: running [finetune] with %s", want)
            self.config["load_checkpoint"], self.finetune = str(want), True
            return
        if self.model_path:
            found = [f for pat in WEIGHT_PATTERNS for f in sorted(glob.glob(os.path.join(self.model_path, pat)))]
            if found:
                # a directory of (sharded) safetensors loads as a whole; a single file loads by itself
                target = self.model_path if found[0].endswith(".safetensors") and os.path.exists(
                    os.path.join(self.model_path, "config.json")) else found[0]
                self.logger.info("weights found under the model directory: running [finetune] with %s", target)
                self.config["load_checkpoint"], self.finetune = target, True
                return
        self.logger.info("no weights: running [pretrain] from random initialisation")
        self.config["load_checkpoint"] = ""

    # ---- network -----------------------------------------------------------------------------------------------
    def build_model(self):
        from mindformers_b200.models import build_network
        self.logger.info("build base model %s", self.model_name)
        model_section = copy.deepcopy(dict(self.config["model"]))
        pet = (model_section.get("model_config") or {}).pop("pet_config", None)
        self.network = build_network(model_section)
        if self.use_pet_model and pet:
            self.build_pet_model(pet)
        return self.network

    def build_pet_model(self, pet_config):
        from mindformers_b200.pet import get_pet_model
        self.logger.info("build pet model (%s)", dict(pet_config).get("pet_type"))
        self.network = get_pet_model(self.network, dict(pet_config))
