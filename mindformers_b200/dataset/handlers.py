"""Data handlers: turn raw instruction / chat records into token ids, labels and packed sequences.

Reference: ``dataset/handler/*`` (``AlpacaInstructDataHandler``, ``CodeAlpacaInstructDataHandler``,
``AdgenInstructDataHandler``, ``PackingHandler`` with ``actual_seq_len``).
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Callable, Dict, Iterable, List, Optional, Sequence

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
@dataclass
class PackingConfig:
    """Settings of the packing functions (reference ``dataset/handler/packing_handler.py:24``)."""
    seq_length: int = None
    pad_token: int = 0
    ignore_token: int = IGNORE
    seed: int = 42
    dataset_shuffle: bool = False

    def __post_init__(self):
        if self.seq_length is None:
            raise ValueError("seq_length must be set in PackingHandler.")


def pack_examples(dataset: Iterable[Dict[str, Sequence[int]]], config: PackingConfig) -> Dict[str, list]:
    """Sequential packing: samples are appended to the current row until the next one would not fit; samples longer
    than ``seq_length`` are skipped. Inside a row every sample's labels are its own next tokens (``labels[1:]`` plus one
    pad), so no label crosses a sample boundary. Columns: ``input_ids``, ``labels`` (padded to ``seq_length``),
    ``actual_seq_len`` (cumulative sample ends of the row)."""
    out = {"input_ids": [], "labels": [], "actual_seq_len": []}
    ids: List[int] = []
    lab: List[int] = []
    ends: List[int] = []

    def flush():
        gap = config.seq_length - len(ids)
        out["input_ids"].append(ids + [config.pad_token] * gap)
        out["labels"].append(lab + [config.ignore_token] * gap)
        out["actual_seq_len"].append(list(ends))

    for sample in dataset:
        tokens, labels = list(sample["input_ids"]), list(sample["labels"])
        n = len(tokens)
        if n > config.seq_length:
            continue
        if len(ids) + n > config.seq_length:
            flush()
            ids, lab, ends = [], [], []
        ids += tokens
        lab += labels[1:] + [config.pad_token]
        ends.append((ends[-1] if ends else 0) + n)
    if ids:
        flush()
    return out


def truncate_examples(examples: Dict[str, List[Sequence[int]]], config: PackingConfig) -> Dict[str, list]:
    """Truncate mode: all samples of the batch are joined into one stream per column and cut into rows of
    ``seq_length`` (a sample may continue in the next row); the last row is padded. ``actual_seq_len`` lists, per row,
    the lengths of the pieces it holds."""
    L = config.seq_length
    first = next(iter(examples))
    pieces: List[List[int]] = [[]]
    used = 0
    for n in (len(x) for x in examples[first]):
        while used + n > L:
            part = L - used
            if part:
                pieces[-1].append(part)
            pieces.append([])
            n -= part
            used = 0
        if n:
            pieces[-1].append(n)
            used += n
    out = {}
    for key, column in examples.items():
        stream = [t for row in column for t in row]
        rows = [stream[i:i + L] for i in range(0, len(stream), L)] or [[]]
        fill = config.pad_token if key == "input_ids" else config.ignore_token
        rows[-1] = rows[-1] + [fill] * (L - len(rows[-1]))
        out[key] = rows
    out["actual_seq_len"] = [p for p in pieces if p][: len(out[first])]
    return out


class PackingHandler:
    """Packing of tokenised samples into rows of ``seq_length`` tokens: ``pack_strategy="pack"`` places every sample
    whole into the first row with room (first fit; the reference fills rows in order, ``pack_examples`` above does that),
    ``"truncate"`` joins all samples and cuts the stream into rows (``truncate_examples``).

    Output rows carry ``input_ids``, ``labels`` (first token of every packed sample masked) and
    ``actual_seq_len`` (cumulative boundaries, padded with ``seq_length``), the inputs of TND-layout attention.
    """

    def __init__(self, seq_length: int, pack_strategy: str = "pack", pad_token_id: int = 0,
                 ignore_token_id: int = IGNORE, max_segments: int = 128, **kw):
        if pack_strategy not in ("pack", "truncate"):
            raise ValueError("pack_strategy must be 'pack' or 'truncate'")
        self.seq_length, self.strategy = seq_length, pack_strategy
        self.pad, self.ignore, self.max_segments = pad_token_id, ignore_token_id, max_segments

    def _handle_truncate(self, samples):
        cfg = PackingConfig(seq_length=self.seq_length, pad_token=self.pad, ignore_token=self.ignore)
        cols = {"input_ids": [], "labels": []}
        for s in samples:
            ids = [int(t) for t in s["input_ids"]]
            cols["input_ids"].append(ids)
            cols["labels"].append([int(t) for t in s.get("labels", ids)])
        if not cols["input_ids"]:
            return []
        cut = truncate_examples(cols, cfg)
        out = []
        for ids, lab, lens in zip(cut["input_ids"], cut["labels"], cut["actual_seq_len"]):
            asl = np.full(self.max_segments, self.seq_length, dtype=np.int32)
            bounds = np.cumsum(lens)[: self.max_segments]
            asl[: len(bounds)] = bounds
            out.append({"input_ids": np.asarray(ids, dtype=np.int64), "labels": np.asarray(lab, dtype=np.int64), "actual_seq_len": asl})
        return out

    def handle(self, samples: Iterable[Dict[str, np.ndarray]]) -> List[Dict[str, np.ndarray]]:
        if self.strategy == "truncate":
            return self._handle_truncate(samples)
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
