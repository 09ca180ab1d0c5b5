"""Data handlers: turn raw instruction / chat records into token ids, labels and packed sequences.

Reference: ``dataset/handler/*`` (``AlpacaInstructDataHandler``, ``CodeAlpacaInstructDataHandler``,
``AdgenInstructDataHandler``, ``PackingHandler`` with ``actual_seq_len``).
"""
from __future__ import annotations

import os
from typing import Callable, Dict, Iterable, List, Optional

import numpy as np

from ..tools.register import MindFormerModuleType, MindFormerRegister

IGNORE = -100

ALPACA_WITH_INPUT = ("Below is an instruction that describes a task, paired with an input that provides further "
                     "context. Write a response that appropriately completes the request.\n\n"
                     "### Instruction:\n{instruction}\n\n### Input:\n{input}\n\n### Response:\n")
ALPACA_NO_INPUT = ("Below is an instruction that describes a task. Write a response that appropriately completes "
                   "the request.\n\n### Instruction:\n{instruction}\n\n### Response:\n")


class BaseInstructDataHandler:
    """Tokenise (prompt, answer) pairs; prompt positions are masked out of the loss."""

    def __init__(self, tokenizer=None, seq_length: int = 2048, padding: bool = True, ignore_token_id: int = IGNORE,
                 prompt_key: str = "instruction", output_columns=None, **kw):
        self.tokenizer, self.seq_length, self.padding = tokenizer, seq_length, padding
        self.ignore = ignore_token_id

    def format(self, record: dict):
        raise NotImplementedError

    def encode(self, text: str) -> List[int]:
        if callable(getattr(self.tokenizer, "encode", None)):
            return list(self.tokenizer.encode(text, add_special_tokens=False))
        return list(self.tokenizer(text))

    def handle_one(self, record: dict) -> Dict[str, np.ndarray]:
        prompt, answer = self.format(record)
        p, a = self.encode(prompt), self.encode(answer)
        eos = getattr(self.tokenizer, "eos_token_id", None)
        if eos is not None:
            a = a + [eos]
        ids = (p + a)[: self.seq_length + 1]
        labels = ([self.ignore] * len(p) + a)[: self.seq_length + 1]
        if self.padding:
            pad = getattr(self.tokenizer, "pad_token_id", 0) or 0
            ids = ids + [pad] * (self.seq_length + 1 - len(ids))
            labels = labels + [self.ignore] * (self.seq_length + 1 - len(labels))
        return {"input_ids": np.asarray(ids, dtype=np.int64), "labels": np.asarray(labels, dtype=np.int64)}

    def handle(self, records: Iterable[dict]) -> List[Dict[str, np.ndarray]]:
        return [self.handle_one(r) for r in records]


@MindFormerRegister.register(MindFormerModuleType.DATA_HANDLER)
class AlpacaInstructDataHandler(BaseInstructDataHandler):
    """Alpaca records (``instruction``, optional ``input``, ``output``) rendered with the Alpaca prompt; only the
    response carries loss."""

    def format(self, r):
        tpl = ALPACA_WITH_INPUT if r.get("input") else ALPACA_NO_INPUT
        return tpl.format(instruction=r.get("instruction", ""), input=r.get("input", "")), r.get("output", "")


@MindFormerRegister.register(MindFormerModuleType.DATA_HANDLER)
class CodeAlpacaInstructDataHandler(AlpacaInstructDataHandler):
    """Code-Alpaca records: the Alpaca format."""

    pass


@MindFormerRegister.register(MindFormerModuleType.DATA_HANDLER)
class AdgenInstructDataHandler(BaseInstructDataHandler):
    """ADGEN records: ``content`` is the prompt, ``summary`` the target."""

    def format(self, r):
        return r.get("content", ""), r.get("summary", "")


@MindFormerRegister.register(MindFormerModuleType.DATA_HANDLER)
class LlavaInstructDataHandler(BaseInstructDataHandler):
    """LLaVA-style visual instruction records: ``{"image": "x.jpg", "conversations": [{"from": "human", "value":
    "<image>\n..."}, {"from": "gpt", "value": "..."}, ...]}`` → multi-turn text with the image tag expanded to
    ``image_token_num`` placeholder tokens; only the assistant turns carry loss. ``image_dir`` is prepended to the
    image path, which is kept in the output for the multimodal dataset to load
    (reference ``dataset/handler/llava_handler.py``)."""

    def __init__(self, tokenizer=None, seq_length: int = 2048, image_dir: str = "", image_token: str = "<image>",
                 image_token_num: int = 1, user_prefix: str = "USER: ", assistant_prefix: str = " ASSISTANT: ", **kw):
        super().__init__(tokenizer, seq_length, **kw)
        self.image_dir, self.image_token, self.image_token_num = image_dir, image_token, max(1, image_token_num)
        self.user_prefix, self.assistant_prefix = user_prefix, assistant_prefix

    def format(self, r):
        raise NotImplementedError("multi-turn records are handled as a whole by handle_one")

    def handle_one(self, record: dict) -> Dict[str, np.ndarray]:
        ids: List[int] = []
        labels: List[int] = []
        eos = getattr(self.tokenizer, "eos_token_id", None)
        for turn in record.get("conversations", []):
            human = turn.get("from") in ("human", "user")
            text = turn.get("value", "").replace(self.image_token, self.image_token * self.image_token_num)
            piece = self.encode((self.user_prefix if human else self.assistant_prefix) + text)
            if not human and eos is not None:
                piece = piece + [eos]
            ids += piece
            labels += [self.ignore] * len(piece) if human else piece
        ids, labels = ids[: self.seq_length + 1], labels[: self.seq_length + 1]
        if self.padding:
            pad = getattr(self.tokenizer, "pad_token_id", 0) or 0
            ids = ids + [pad] * (self.seq_length + 1 - len(ids))
            labels = labels + [self.ignore] * (self.seq_length + 1 - len(labels))
        out = {"input_ids": np.asarray(ids, dtype=np.int64), "labels": np.asarray(labels, dtype=np.int64)}
        if record.get("image"):
            out["image_path"] = os.path.join(self.image_dir, record["image"]) if self.image_dir else record["image"]
        return out


@MindFormerRegister.register(MindFormerModuleType.DATA_HANDLER)
class PackingHandler:
    """Greedy first-fit packing of tokenised samples into rows of ``seq_length`` tokens.

    Output rows carry ``input_ids``, ``labels`` (first token of every packed sample masked) and
    ``actual_seq_len`` (cumulative boundaries, padded with ``seq_length``), the inputs of TND-layout attention.
    """

    def __init__(self, seq_length: int, pack_strategy: str = "pack", pad_token_id: int = 0,
                 ignore_token_id: int = IGNORE, max_segments: int = 128, **kw):
        if pack_strategy not in ("pack", "truncate"):
            raise ValueError("pack_strategy must be 'pack' or 'truncate'")
        self.seq_length, self.strategy = seq_length, pack_strategy
        self.pad, self.ignore, self.max_segments = pad_token_id, ignore_token_id, max_segments

    def handle(self, samples: Iterable[Dict[str, np.ndarray]]) -> List[Dict[str, np.ndarray]]:
        rows: List[List[Dict[str, np.ndarray]]] = []
        space: List[int] = []
        for s in samples:
            ids = np.asarray(s["input_ids"])
            lab = np.asarray(s.get("labels", ids))
            n = min(len(ids), self.seq_length)
            item = {"input_ids": ids[:n], "labels": lab[:n]}
            placed = False
            if self.strategy == "pack":
                for i, free in enumerate(space):
                    if free >= n and len(rows[i]) < self.max_segments:
                        rows[i].append(item)
                        space[i] -= n
                        placed = True
                        break
            if not placed:
                rows.append([item])
                space.append(self.seq_length - n)
        out = []
        for items in rows:
            ids = np.full(self.seq_length, self.pad, dtype=np.int64)
            lab = np.full(self.seq_length, self.ignore, dtype=np.int64)
            bounds, pos = [], 0
            for it in items:
                n = len(it["input_ids"])
                ids[pos:pos + n] = it["input_ids"]
                lab[pos:pos + n] = it["labels"]
                lab[pos] = self.ignore if pos > 0 else lab[pos]
                pos += n
                bounds.append(pos)
            asl = np.full(self.max_segments, self.seq_length, dtype=np.int32)
            asl[: len(bounds)] = bounds
            out.append({"input_ids": ids, "labels": lab, "actual_seq_len": asl})
        return out


def build_data_handler(config: Optional[dict] = None, default_args: Optional[dict] = None, **kwargs):
    if config is None:
        return None
    cfg = dict(config)
    cfg.update(kwargs)
    return MindFormerRegister.get_instance_from_cfg(cfg, MindFormerModuleType.DATA_HANDLER, default_args=default_args)
