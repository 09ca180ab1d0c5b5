"""Tokenizer helpers: a dependency-free byte-level tokenizer and the text processor used by pipelines.

Real models use their HF tokenizer files through ``AutoTokenizer`` (the reference vendors HF's tokenizer base
classes, ``models/tokenization_utils*.py``); ``ByteTokenizer`` gives tests and ``run_check`` a vocabulary of 256
bytes + specials without any file.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Union

from ..tools.register import MindFormerModuleType, MindFormerRegister


@MindFormerRegister.register(MindFormerModuleType.TOKENIZER)
class ByteTokenizer:
    """Tokenizer without a vocabulary file: UTF-8 bytes shifted past the special ids. Used by tests, ``run_check``
    and as the fallback when a model directory has no tokenizer."""

    pad_token, bos_token, eos_token, unk_token = "<pad>", "<s>", "</s>", "<unk>"

    def __init__(self, add_bos_token: bool = True, add_eos_token: bool = False, **kw):
        self.pad_token_id, self.bos_token_id, self.eos_token_id, self.unk_token_id = 0, 1, 2, 3
        self.offset = 4
        self.vocab_size = 256 + self.offset
        self.add_bos_token, self.add_eos_token = add_bos_token, add_eos_token
        self.chat_template = None

    def __len__(self):
        return self.vocab_size

    def tokenize(self, text: str) -> List[str]:
        return [chr(b) for b in text.encode("utf-8")]

    def encode(self, text: str, add_special_tokens: bool = True, **kw) -> List[int]:
        ids = [b + self.offset for b in text.encode("utf-8")]
        if add_special_tokens and self.add_bos_token:
            ids = [self.bos_token_id] + ids
        if add_special_tokens and self.add_eos_token:
            ids = ids + [self.eos_token_id]
        return ids

    def decode(self, ids: Sequence[int], skip_special_tokens: bool = True, **kw) -> str:
        if hasattr(ids, "tolist"):
            ids = ids.tolist()
        data = bytes(i - self.offset for i in ids if i >= self.offset and i < self.vocab_size)
        text = data.decode("utf-8", errors="replace")
        if not skip_special_tokens:
            specials = {0: self.pad_token, 1: self.bos_token, 2: self.eos_token, 3: self.unk_token}
            text = "".join(specials.get(i, "") for i in ids if i < self.offset) + text
        return text

    def batch_decode(self, batch, **kw) -> List[str]:
        return [self.decode(x, **kw) for x in batch]

    def __call__(self, text: Union[str, List[str]], padding: bool = False, max_length: Optional[int] = None,
                 truncation: bool = False, add_special_tokens: bool = True, return_tensors: Optional[str] = None, **kw):
        single = isinstance(text, str)
        rows = [self.encode(t, add_special_tokens) for t in ([text] if single else text)]
        if truncation and max_length:
            rows = [r[:max_length] for r in rows]
        mask = [[1] * len(r) for r in rows]
        if padding:
            width = max_length if padding == "max_length" and max_length else max(len(r) for r in rows)
            mask = [m + [0] * (width - len(m)) for m in mask]
            rows = [r + [self.pad_token_id] * (width - len(r)) for r in rows]
        out = {"input_ids": rows[0] if single and not return_tensors else rows,
               "attention_mask": mask[0] if single and not return_tensors else mask}
        if return_tensors == "pt":
            import torch
            out = {k: torch.tensor(v) for k, v in out.items()}
        return out

    def save_pretrained(self, directory: str):
        import json
        import os
        os.makedirs(directory, exist_ok=True)
        with open(os.path.join(directory, "tokenizer_config.json"), "w") as f:
            json.dump({"tokenizer_class": "ByteTokenizer", "add_bos_token": self.add_bos_token}, f)


@MindFormerRegister.register(MindFormerModuleType.PROCESSOR)
class TextProcessor:
    """Tokenise raw text into padded id batches (the text part of the reference's ``ProcessorMixin``)."""

    def __init__(self, tokenizer=None, max_length: int = 128, padding: str = "max_length", return_tensors: str = "pt", **kw):
        self.tokenizer, self.max_length, self.padding, self.return_tensors = tokenizer, max_length, padding, return_tensors

    def __call__(self, text_input=None, **kw):
        enc = self.tokenizer(text_input, padding=self.padding, max_length=self.max_length, truncation=True,
                             return_tensors=self.return_tensors)
        return {"text": enc["input_ids"], "attention_mask": enc.get("attention_mask")}


def build_tokenizer(config: Optional[dict] = None, **kwargs):
    """``{"type": "ByteTokenizer"}`` from the registry, or ``{"pretrained_model_dir"|"vocab_file": path}`` via HF."""
    if config is None:
        return None
    cfg = dict(config)
    cfg.update(kwargs)
    path = cfg.pop("pretrained_model_dir", None) or cfg.pop("tokenizer_dir", None)
    if path:
        from .auto import AutoTokenizer
        return AutoTokenizer.from_pretrained(path)
    if "type" in cfg and MindFormerRegister.is_exist(MindFormerModuleType.TOKENIZER, cfg["type"]):
        return MindFormerRegister.get_instance_from_cfg(cfg, MindFormerModuleType.TOKENIZER)
    raise ValueError(f"cannot build a tokenizer from {config!r}")
