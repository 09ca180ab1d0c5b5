"""``run_check()``: installation sanity check (``mindformers/run_check.py:108,366``): versions, the kernel library,
then a 2-layer Llama trained for a few steps and used for a short generation. Prints one verdict line per stage."""
from __future__ import annotations

import json
import os
import tempfile
import time

import torch

from .tools.logger import get_logger

logger = get_logger()
VERSION = "1.6.0+b200"


class MFCheck:
    """Installation self-check (reference ``mindformers/run_check.py:108``): version line, kernel library, a two-layer
    Llama trained for a few steps, a short generation; prints one verdict per stage."""

    def __init__(self, steps: int = 3, device: str = None):
        self.steps = steps
        self.device = device or ("cuda" if torch.cuda.is_available() else "cpu")
        self.results = {}

    def _stage(self, name, fn):
        t0 = time.time()
        try:
            out = fn()
            self.results[name] = {"ok": True, "seconds": round(time.time() - t0, 2), "detail": out}
            logger.info("[run_check] %-18s passed (%.1fs) %s", name, time.time() - t0, out if out is not None else "")
        except Exception as e:  # noqa: BLE001 - the check reports every failure
            self.results[name] = {"ok": False, "error": f"{type(e).__name__}: {e}"}
            logger.error("[run_check] %-18s FAILED: %s", name, e)

    @staticmethod
    def version_map() -> dict:
        """``VERSION_MAP.json`` next to the package: framework version -> supported torch / CUDA versions (the
        reference keeps the same table for MindSpore versions)."""
        import json
        import os
        with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "VERSION_MAP.json")) as f:
            return json.load(f)["mindformers_b200"]

    def check_versions(self):
        from . import __version__
        info = {"framework": VERSION, "package": __version__, "torch": torch.__version__, "cuda": torch.version.cuda,
                "device": torch.cuda.get_device_name(0) if torch.cuda.is_available() else "cpu"}
        entry = self.version_map().get(__version__)
        if entry is None:
            raise RuntimeError(f"VERSION_MAP.json has no entry for package version {__version__}")
        tv = ".".join(torch.__version__.split("+")[0].split(".")[:2])
        info["torch_supported"] = tv in entry["torch"]["support"]
        if not info["torch_supported"]:
            logger.warning("[run_check] torch %s is outside the tested range %s (preferred %s)", tv,
                           entry["torch"]["support"], entry["torch"]["prefer"])
        if torch.version.cuda and torch.cuda.is_available():
            info["cuda_supported"] = ".".join(torch.version.cuda.split(".")[:2]) in entry["cuda"]["support"]
        if torch.cuda.is_available():
            major, minor = torch.cuda.get_device_capability(0)
            info["sm"] = f"{major}{minor}"
            if major != 10:
                raise RuntimeError(f"the kernel library targets sm_100a; found sm_{major}{minor}")
        return info

    def check_kernel_library(self):
        from .ops import _lib
        if not _lib.available():
            if self.device == "cuda":
                raise RuntimeError("kernel library missing: run `python -m mindformers_b200.ops.build`")
            return "not built (CPU only)"
        return f"abi {_lib.get_lib().mfb_abi_version()}"

    def _config(self, out):
        dt = "bfloat16" if self.device == "cuda" else "float32"
        return dict(output_dir=out, run_mode="train", use_legacy=False, seed=0,
                    model=dict(arch=dict(type="LlamaForCausalLM"),
                               model_config=dict(model_type="llama", vocab_size=512, hidden_size=256, intermediate_size=512,
                                                 num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, seq_length=128,
                                                 max_position_embeddings=128, params_dtype=dt, compute_dtype=dt)),
                    runner_config=dict(epochs=1, batch_size=2, stop_step=self.steps),
                    train_dataset=dict(data_loader=dict(type="MockDataLoader", num_samples=64, seq_length=128, vocab_size=512)),
                    train_dataset_task=dict(type="CausalLanguageModelDataset"),
                    optimizer=dict(type="AdamW", learning_rate=1e-3), context=dict(device_target="CUDA" if self.device == "cuda" else "CPU"),
                    lr_schedule=dict(type="ConstantWarmUpLR", learning_rate=1e-3, warmup_steps=0, total_steps=-1),
                    callbacks=[dict(type="MFLossMonitor")])

    def check_train_and_predict(self):
        from .core import context
        from .trainer import Trainer
        context._CONTEXT = None
        with tempfile.TemporaryDirectory() as out:
            t = Trainer(args=self._config(out))
            t.train()
            losses = t.trainer.loss_history
            if len(losses) != self.steps or not all(l == l for l in losses):
                raise RuntimeError(f"training produced {losses}")
            from .models import LlamaConfig, LlamaForCausalLM
            mc = self._config(out)["model"]["model_config"]
            mc.pop("model_type")
            net = LlamaForCausalLM(LlamaConfig(**mc), device=self.device)
            toks = net.generate([[1, 2, 3, 4]], max_new_tokens=4)[0]
            if len(toks) != 8:
                raise RuntimeError(f"generation returned {toks}")
            return {"losses": [round(x, 4) for x in losses], "generated": toks}

    def check(self) -> bool:
        self._stage("versions", self.check_versions)
        self._stage("kernel library", self.check_kernel_library)
        self._stage("train + predict", self.check_train_and_predict)
        ok = all(r["ok"] for r in self.results.values())
        logger.info("[run_check] %s", "All checks passed, the installation works." if ok else "Some checks FAILED.")
        return ok


def run_check(log_level: str = "info") -> bool:
    """Installation self-check (reference ``mindformers/run_check.py:366``): returns True when every stage passed."""

    return MFCheck().check()


if __name__ == "__main__":
    import sys
    sys.exit(0 if run_check() else 1)
