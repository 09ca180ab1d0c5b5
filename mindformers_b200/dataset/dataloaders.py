"""Record-level data loaders for supervised fine-tuning and raw-text pre-training.

Each loader is a registry entry (``MindFormerModuleType.DATASET_LOADER``) that returns a map-style (or iterable)
dataset of dict rows; ``CausalLanguageModelDataset`` / ``KeyWordGenDataset`` / ``MultiTurnDataset`` shard, batch and
collate them. They cover the reference's ``dataset/dataloader`` package:

* ``SFTDataLoader``        json / jsonl / parquet / csv / tsv records → tokenised ``input_ids`` / ``labels`` through a
                           named map function (``sft_dataloader.py``, ``sft_map_functions.py``).
* ``ADGenDataLoader``      AdvertiseGen ``{"content", "summary"}`` lines (``adgen_dataloader.py``).
* ``ToolAlpacaDataLoader`` ToolAlpaca conversations with validity checks (``toolaplaca_dataloader.py``).
* ``MultiSourceDataLoader`` several sub-loaders mixed by sample counts or ratios, with an optional shuffle buffer
                           (``multi_source_dataloader.py``).
* ``TrainingDataLoader``   text files → tokenise → concatenate → fixed-length samples (``training_dataloader.py``).
"""
from __future__ import annotations

import csv
import glob
import json
import os
import random
from typing import Callable, Dict, Iterable, List, Optional, Sequence, Union

import numpy as np
import torch
from torch.utils.data import Dataset, IterableDataset

from ..tools.register import MindFormerModuleType, MindFormerRegister

IGNORE_INDEX = -100


# ---- file readers ----------------------------------------------------------------------------------
def read_records(path: str, file_format: Optional[str] = None) -> List[dict]:
    """Rows of one file as dicts. ``json`` holds a list or one object per line; parquet/csv/tsv go through pyarrow."""
    fmt = (file_format or os.path.splitext(path)[1].lstrip(".")).lower()
    if fmt in ("json", "jsonl"):
        with open(path, "r", encoding="utf-8") as f:
            text = f.read().strip()
        if not text:
            return []
        if text[0] == "[":
            return list(json.loads(text))
        return [json.loads(line) for line in text.splitlines() if line.strip()]
    if fmt == "parquet":
        import pyarrow.parquet as pq
        return pq.read_table(path).to_pylist()
    if fmt in ("csv", "tsv"):
        with open(path, "r", encoding="utf-8", newline="") as f:
            return list(csv.DictReader(f, delimiter="\t" if fmt == "tsv" else ","))
    if fmt in ("txt", "text"):
        with open(path, "r", encoding="utf-8") as f:
            return [{"text": line.rstrip("\n")} for line in f if line.strip()]
    raise ValueError(f"unsupported file format {fmt!r} for {path}")


def list_files(dataset_dir: str, file_format: Optional[str] = None) -> List[str]:
    if os.path.isfile(dataset_dir):
        return [dataset_dir]
    exts = [file_format] if file_format else ["json", "jsonl", "parquet", "csv", "tsv", "txt"]
    files: List[str] = []
    for e in exts:
        files += glob.glob(os.path.join(dataset_dir, "**", f"*.{e}"), recursive=True)
    if not files:
        raise FileNotFoundError(f"no {exts} files under {dataset_dir}")
    return sorted(files)


def cmrc2018_reader(path: str) -> List[dict]:
    """SQuAD-style CMRC2018 json → ``{"prompt", "answer"}`` rows (reference ``datareaders.py:21``)."""
    with open(path, "r", encoding="utf-8") as f:
        data = json.load(f)["data"]
    rows = []
    for doc in data:
        for para in doc["paragraphs"]:
            for qa in para["qas"]:
                rows.append({"prompt": f"阅读文章：{para['context']}\n问：{qa['question']}\n答：",
                             "answer": qa["answers"][0]["text"] if qa["answers"] else ""})
    return rows


def wikitext_reader(path: str) -> List[dict]:
    """WikiText raw file → one row per article, spacing around punctuation repaired (``datareaders.py:40``)."""
    import re
    with open(path, "r", encoding="utf-8") as f:
        text = f.read()
    for a, b in ((" @-@ ", "-"), (" @,@ ", ","), (" @.@ ", "."), (" , ", ", "), (" . ", ". "), (" ; ", "; "),
                 (" : ", ": "), (" 's", "'s"), ("( ", "("), (" )", ")"), (" n't", "n't")):
        text = text.replace(a, b)
    parts = re.split(r"\n \= [^=\n]+ \= \n", "\n" + text)
    return [{"text": p.strip()} for p in parts if p.strip()]


DATA_READERS: Dict[str, Callable[[str], List[dict]]] = {"cmrc2018": cmrc2018_reader, "wikitext": wikitext_reader}


# ---- map functions ---------------------------------------------------------------------------------
def _ids(tokenizer, text: str) -> List[int]:
    return list(tokenizer.encode(text, add_special_tokens=False))


def prepare_for_model(tokenizer, max_length: int, prompt: str, answer: Optional[str] = None) -> Dict[str, List[int]]:
    """``bos + prompt + answer + eos`` cut to ``max_length``; labels ignore the prompt."""
    bos = [tokenizer.bos_token_id] if getattr(tokenizer, "bos_token_id", None) is not None and getattr(
        tokenizer, "add_bos_token", True) else []
    p = bos + _ids(tokenizer, prompt)
    a = (_ids(tokenizer, answer) + [tokenizer.eos_token_id]) if answer is not None else []
    ids = (p + a)[:max_length]
    labels = ([IGNORE_INDEX] * len(p) + a)[:max_length]
    return {"input_ids": ids, "labels": labels}


def default_map_fn(example, tokenizer, max_length, prompt_key="prompt", answer_key="answer", **kw):
    return prepare_for_model(tokenizer, max_length, str(example[prompt_key]), str(example.get(answer_key, "")))


ALPACA_WITH_INPUT = ("Below is an instruction that describes a task, paired with an input that provides further context. "
                     "Write a response that appropriately completes the request.\n\n"
                     "### Instruction:\n{instruction}\n\n### Input:\n{input}\n\n### Response:\n")
ALPACA_NO_INPUT = ("Below is an instruction that describes a task. "
                   "Write a response that appropriately completes the request.\n\n"
                   "### Instruction:\n{instruction}\n\n### Response:\n")


def alpaca_map_fn(example, tokenizer, max_length, **kw):
    tmpl = ALPACA_WITH_INPUT if example.get("input") else ALPACA_NO_INPUT
    return prepare_for_model(tokenizer, max_length, tmpl.format(**{"input": "", **example}), str(example["output"]))


def advertisegen_map_fn(example, tokenizer, max_length, **kw):
    return prepare_for_model(tokenizer, max_length, str(example["content"]), str(example["summary"]))


def tnews_map_fn(example, tokenizer, max_length, label_names: Optional[Sequence[str]] = None, **kw):
    label = example.get("label_desc", example.get("label"))
    if label_names is not None and str(label).isdigit():
        label = label_names[int(label)]
    prompt = f"新闻：{example['sentence']}\n这条新闻的类别是："
    return prepare_for_model(tokenizer, max_length, prompt, str(label))


def multi_round_chat_map_fn(example, tokenizer, max_length, user_role="human", assistant_role="gpt",
                            user_prefix="<|user|>\n", assistant_prefix="<|assistant|>\n", system_prefix="<|system|>\n",
                            **kw):
    """``{"conversations": [{"from", "value"}, …]}``; only assistant turns carry loss."""
    ids: List[int] = []
    labels: List[int] = []
    if getattr(tokenizer, "bos_token_id", None) is not None and getattr(tokenizer, "add_bos_token", True):
        ids.append(tokenizer.bos_token_id)
        labels.append(IGNORE_INDEX)
    for turn in example["conversations"]:
        role, value = turn.get("from", turn.get("role")), turn.get("value", turn.get("content", ""))
        if role in (assistant_role, "assistant"):
            head = _ids(tokenizer, assistant_prefix)
            body = _ids(tokenizer, value) + [tokenizer.eos_token_id]
            ids += head + body
            labels += [IGNORE_INDEX] * len(head) + body
        else:
            prefix = system_prefix if role == "system" else user_prefix
            part = _ids(tokenizer, prefix + value + "\n")
            ids += part
            labels += [IGNORE_INDEX] * len(part)
    return {"input_ids": ids[:max_length], "labels": labels[:max_length]}


def _dyn_row(ids: List[int], labels: List[int], tokenizer, max_length: int) -> Dict[str, List[int]]:
    """Close a dynamic-length row: append the end token, cut at ``max_length``; no padding (the batch collator pads)."""
    ids, labels = ids + [tokenizer.eos_token_id], labels + [tokenizer.eos_token_id]
    ids, labels = ids[:max_length], labels[:max_length]
    return {"input_ids": ids, "attention_mask": [1] * len(ids), "labels": labels}


def _chat_turns(example, kw):
    field = kw.get("data_field", "conversations")
    fk, vk = kw.get("from_keyword", "from"), kw.get("value_keyword", "value")
    user, assistant = kw.get("user_role_name", "human"), kw.get("assistant_role_name", "gpt")
    for message in example[field]:
        role = message[fk]
        if role not in (user, assistant):
            raise ValueError(f"Incorrect role name: {role}. Check the values of `user_role_name` and `assistant_role_name` "
                             f"in `map_function_kwargs`.")
        yield role == user, message[vk]


def multi_round_chat_dyn_map_fn(example, tokenizer=None, max_length=None, **kw):
    """Multi-round chat without padding (reference ``sft_map_functions.py:119``): a user turn is ``bos_token + user_prompt
    + user_prompt_role + text`` followed by ``assistant_prompt + assistant_prompt_role`` (no loss); an assistant turn is
    ``sep_token + text`` (loss on all of it); one end token closes the row."""
    ignore = kw.get("ignore_token_id", IGNORE_INDEX)
    bos, sep = kw.get("bos_token", "<s>"), kw.get("sep_token", "")
    ids: List[int] = []
    labels: List[int] = []
    for is_user, text in _chat_turns(example, kw):
        if is_user:
            part = _ids(tokenizer, bos + kw.get("user_prompt", "") + kw.get("user_prompt_role", "") + text) + \
                _ids(tokenizer, kw.get("assistant_prompt", "") + kw.get("assistant_prompt_role", ""))
            ids += part
            labels += [ignore] * len(part)
        else:
            part = _ids(tokenizer, sep + text)
            ids += part
            labels += part
    return _dyn_row(ids, labels, tokenizer, max_length)


def multi_instruct_dyn_map_fn(example, tokenizer=None, max_length=None, **kw):
    """Instruction / input / output records without padding (reference ``sft_map_functions.py:166``): the prompt
    ``user_prompt_role + instruction + input + assistant_prompt_role`` carries no loss, the output does."""
    ignore = kw.get("ignore_token_id", IGNORE_INDEX)
    prompt = _ids(tokenizer, kw.get("user_prompt_role", "") + example[kw.get("instruction_keyword", "instruction")]
                  + example[kw.get("from_keyword", "input")] + kw.get("assistant_prompt_role", ""))
    answer = _ids(tokenizer, example[kw.get("value_keyword", "output")])
    return _dyn_row(prompt + answer, [ignore] * len(prompt) + answer, tokenizer, max_length)


def multi_round_chat_dyn_map_fn_alpaca(example, tokenizer=None, max_length=None, **kw):
    """ChatML-formatted multi-round chat without padding (reference ``sft_map_functions.py:204``): user turns are
    ``bos + user_prompt + sep + user_prompt_role + text + sep`` + the assistant prompt, assistant turns end with
    ``<|im_end|>\\n``; every token carries loss (continued pre-training on chat transcripts)."""
    bos, sep = kw.get("bos_token", "<|im_start|>"), kw.get("sep_token", "<|im_end|>\n<|im_start|>")
    ids: List[int] = []
    for is_user, text in _chat_turns(example, kw):
        if is_user:
            ids += _ids(tokenizer, bos + kw.get("user_prompt", "") + sep + kw.get("user_prompt_role", "") + text + sep)
            ids += _ids(tokenizer, kw.get("assistant_prompt", "") + kw.get("assistant_prompt_role", ""))
        else:
            ids += _ids(tokenizer, text + "<|im_end|>\n")
    return _dyn_row(ids, list(ids), tokenizer, max_length)


SFT_MAP_FUNCTIONS: Dict[str, Callable] = {
    "default": default_map_fn, "alpaca": alpaca_map_fn, "advertisegen": advertisegen_map_fn, "tnews": tnews_map_fn,
    "cmrc2018": default_map_fn, "multi-round-chat": multi_round_chat_map_fn,
    "multi-round-chat-dyn": multi_round_chat_dyn_map_fn, "multi-instruct-dyn": multi_instruct_dyn_map_fn,
    "multi-round-chat-dyn-alpaca": multi_round_chat_dyn_map_fn_alpaca,
}


def _resolve_tokenizer(tokenizer):
    if isinstance(tokenizer, (dict, str)):
        from ..models.tokenization import build_tokenizer
        return build_tokenizer({"pretrained_model_dir": tokenizer} if isinstance(tokenizer, str) else tokenizer)
    return tokenizer


def _finish(row: Dict[str, List[int]], max_length: int, pad_id: int, pad: bool) -> Dict[str, torch.Tensor]:
    """Shift labels by one (position ``t`` predicts token ``t+1``) and optionally pad to ``max_length - 1``."""
    ids, labels = row["input_ids"], row["labels"]
    ids, labels = ids[:-1], labels[1:]
    if pad:
        gap = (max_length - 1) - len(ids)
        ids, labels = ids + [pad_id] * gap, labels + [IGNORE_INDEX] * gap
    mask = [0 if l == IGNORE_INDEX else 1 for l in labels]
    return {"input_ids": torch.tensor(ids, dtype=torch.int64), "labels": torch.tensor(labels, dtype=torch.int64),
            "loss_mask": torch.tensor(mask, dtype=torch.float32)}


class _MappedRecords(Dataset):
    def __init__(self, records: List[dict], fn: Callable, tokenizer, max_length: int, pad: bool, fn_kwargs: dict):
        self.records, self.fn, self.tokenizer = records, fn, tokenizer
        self.max_length, self.pad, self.fn_kwargs = max_length, pad, fn_kwargs
        pid = getattr(tokenizer, "pad_token_id", None)
        self.pad_id = 0 if pid is None else pid

    def __len__(self):
        return len(self.records)

    def __getitem__(self, i):
        row = self.fn(self.records[i], tokenizer=self.tokenizer, max_length=self.max_length, **self.fn_kwargs)
        return _finish(row, self.max_length, self.pad_id, self.pad)


@MindFormerRegister.register(MindFormerModuleType.DATASET_LOADER)
class SFTDataLoader:
    """``max_length`` counts the unshifted sequence: rows come out with ``max_length - 1`` positions."""

    def __new__(cls, dataset_dir: str, tokenizer, dataset_name: str = "", file_format: Optional[str] = None,
                max_length: int = 1025, read_function: Optional[Callable] = None,
                map_function: Optional[Callable] = None, map_function_kwargs: Optional[dict] = None,
                shuffle: bool = False, seed: int = 0, pad_to_max_length: bool = True, column_names=None, **kw):
        reader = read_function or DATA_READERS.get(dataset_name)
        records: List[dict] = []
        for path in list_files(dataset_dir, file_format):
            records += reader(path) if reader else read_records(path, file_format)
        if shuffle:
            random.Random(seed).shuffle(records)
        fn = map_function or SFT_MAP_FUNCTIONS.get(dataset_name or "default")
        if fn is None:
            raise ValueError(f"dataset_name {dataset_name!r}: pass map_function or one of {sorted(SFT_MAP_FUNCTIONS)}")
        return _MappedRecords(records, fn, _resolve_tokenizer(tokenizer), int(max_length), pad_to_max_length,
                              dict(map_function_kwargs or {}))


class _RawRecords(Dataset):
    """Untokenised rows; a task dataset (``KeyWordGenDataset`` / ``MultiTurnDataset``) tokenises them."""

    def __init__(self, rows: List[dict]):
        self.rows = rows

    def __len__(self):
        return len(self.rows)

    def __getitem__(self, i):
        return self.rows[i]


@MindFormerRegister.register(MindFormerModuleType.DATASET_LOADER)
class ADGenDataLoader:
    """``{"content": prompt, "summary": answer}`` per line → rows ``{"prompt", "answer"}``."""

    def __new__(cls, dataset_dir: str, phase: str = "train", shuffle: bool = False,
                origin_columns=("content", "summary"), seed: int = 0, **kw):
        if phase not in ("train", "eval"):
            raise ValueError(f"phase must be train or eval, got {phase!r}")
        pk, ak = origin_columns
        rows = []
        for path in list_files(dataset_dir):
            for i, r in enumerate(read_records(path)):
                if pk not in r or ak not in r:
                    raise KeyError(f"{path} row {i}: needs columns {pk!r} and {ak!r}")
                rows.append({"prompt": r[pk], "answer": r[ak]})
        if shuffle:
            random.Random(seed).shuffle(rows)
        return _RawRecords(rows)


@MindFormerRegister.register(MindFormerModuleType.DATASET_LOADER)
class ToolAlpacaDataLoader:
    """ToolAlpaca jsonl: ``{"tools": [...], "conversations": [{"role", "content"}, …]}``. Rows must open with a user
    turn, alternate user → assistant/tool, and close with an assistant turn; others are skipped with a count."""

    def __new__(cls, dataset_dir: str, shuffle: bool = False, seed: int = 0, **kw):
        rows, bad = [], 0
        for path in list_files(dataset_dir):
            for r in read_records(path):
                conv = r.get("conversations") or []
                ok = (len(conv) >= 2 and conv[0].get("role") in ("user", "system")
                      and conv[-1].get("role") == "assistant"
                      and all(c.get("role") in ("system", "user", "assistant", "tool") for c in conv)
                      and all("content" in c or c.get("role") == "tool" for c in conv))
                if ok:
                    rows.append(r)
                else:
                    bad += 1
        if shuffle:
            random.Random(seed).shuffle(rows)
        ds = _RawRecords(rows)
        ds.skipped = bad
        return ds


class MultiSourceDataset(Dataset):
    """Samples of several datasets in one index space.

    ``sample_nums[i]`` rows are taken from dataset ``i`` per epoch (over-sampling wraps around). Without shuffle the
    sources follow one another; with shuffle the order of sources is a seeded permutation over all draws, and rows
    inside a source are permuted too.
    """

    def __init__(self, datasets: List[Dataset], sample_nums: List[int], shuffle: bool = False, seed: int = 0):
        self.datasets = datasets
        rng = np.random.default_rng(seed)
        src = np.concatenate([np.full(n, i, dtype=np.int64) for i, n in enumerate(sample_nums)])
        row = np.concatenate([
            (rng.permutation(max(n, len(d)))[:n] if shuffle else np.arange(n)) % max(len(d), 1)
            for d, n in zip(datasets, sample_nums)])
        if shuffle:
            order = rng.permutation(len(src))
            src, row = src[order], row[order]
        self.src, self.row = src, row

    def __len__(self):
        return len(self.src)

    def __getitem__(self, i):
        return self.datasets[int(self.src[i])][int(self.row[i])]


@MindFormerRegister.register(MindFormerModuleType.DATASET_LOADER)
class MultiSourceDataLoader:
    """``sub_data_loader``: list of loader configs. Mix by ``samples_count`` + ``dataset_ratios`` or by explicit
    ``nums_per_dataset``; default is every row of every source once."""

    def __new__(cls, sub_data_loader: List[dict], sub_data_loader_args: Optional[dict] = None,
                dataset_ratios: Optional[List[float]] = None, samples_count: Optional[int] = None,
                nums_per_dataset: Optional[List[int]] = None, shuffle: bool = False, seed: int = 0, **kw):
        subs = []
        for cfg in sub_data_loader:
            merged = dict(sub_data_loader_args or {})
            merged.update(cfg)
            subs.append(MindFormerRegister.get_instance_from_cfg(merged, MindFormerModuleType.DATASET_LOADER)
                        if isinstance(cfg, dict) else cfg)
        if nums_per_dataset is not None:
            nums = [int(n) for n in nums_per_dataset]
        elif dataset_ratios is not None:
            if abs(sum(dataset_ratios) - 1.0) > 1e-6:
                raise ValueError("dataset_ratios must sum to 1")
            total = samples_count if samples_count is not None else sum(len(d) for d in subs)
            nums = [int(total * r) for r in dataset_ratios]
        else:
            nums = [len(d) for d in subs]
        if len(nums) != len(subs):
            raise ValueError("one sample count per sub loader is required")
        return MultiSourceDataset(subs, nums, shuffle, seed)


class TrainingDataset(IterableDataset):
    """Raw text → fixed-length token samples.

    Files are visited in order (a seeded shuffle of the file list if ``shuffle``); every document is tokenised,
    closed with ``eos`` and appended to a token stream that is cut into ``max_length`` pieces. ``samples_num`` bounds
    the epoch. ``skip_num`` drops the first samples (resume).
    """

    def __init__(self, dataset_dir: str, tokenizer, column_names=("input_ids",), max_length: int = 1025,
                 text_col: str = "text", file_format: Optional[str] = None, shuffle: bool = False, seed: int = 0,
                 samples_num: Optional[int] = None, skip_num: int = 0, file_limit: int = 1,
                 is_align: bool = True):
        self.files = list_files(dataset_dir, file_format)
        if shuffle:
            random.Random(seed).shuffle(self.files)
        self.tokenizer, self.max_length, self.text_col = _resolve_tokenizer(tokenizer), int(max_length), text_col
        self.file_format, self.samples_num, self.skip_num = file_format, samples_num, skip_num
        self.column = column_names[0]
        self.is_align = is_align

    def _documents(self) -> Iterable[str]:
        for path in self.files:
            for r in read_records(path, self.file_format):
                text = r.get(self.text_col)
                if text:
                    yield text

    def __iter__(self):
        buf: List[int] = []
        produced = 0
        eos = self.tokenizer.eos_token_id
        for doc in self._documents():
            buf += list(self.tokenizer.encode(doc, add_special_tokens=False)) + ([eos] if eos is not None else [])
            while len(buf) >= self.max_length:
                piece, buf = buf[:self.max_length], buf[self.max_length:]
                produced += 1
                if produced <= self.skip_num:
                    continue
                yield {self.column: torch.tensor(piece[:-1], dtype=torch.int64),
                       "labels": torch.tensor(piece[1:], dtype=torch.int64)}
                if self.samples_num is not None and produced - self.skip_num >= self.samples_num:
                    return
        if buf and not self.is_align and len(buf) > 1:
            pad = [self.tokenizer.pad_token_id or 0] * (self.max_length - len(buf))
            piece = buf + pad
            labels = buf[1:] + [IGNORE_INDEX] * (len(pad) + 0)
            yield {self.column: torch.tensor(piece[:-1], dtype=torch.int64),
                   "labels": torch.tensor(labels[:self.max_length - 1], dtype=torch.int64)}


@MindFormerRegister.register(MindFormerModuleType.DATASET_LOADER)
class TrainingDataLoader:
    """Text files (plain or JSON lines) tokenised and packed into ``seq_length`` samples on the fly (reference
    ``dataset/dataloader/training_dataloader.py``)."""

    def __new__(cls, dataset_dir: str, tokenizer, column_names=("input_ids",), max_length: int = 1025,
                text_col: str = "text", file_format: Optional[str] = None, shuffle: bool = False,
                samples_num: Optional[int] = None, skip_num: int = 0, **kw):
        return TrainingDataset(dataset_dir, tokenizer, column_names, max_length, text_col, file_format, shuffle,
                               int(kw.get("seed", 0)), samples_num, skip_num, is_align=bool(kw.get("is_align", True)))


class _SampleList(Dataset):
    """Tokenised samples (dicts of int lists / arrays) as tensors, padded or cut to ``seq_length + 1`` and shifted."""

    def __init__(self, samples: List[dict], seq_length: Optional[int], pad_token_id: int = 0):
        self.samples, self.seq_length, self.pad = samples, seq_length, pad_token_id

    def __len__(self):
        return len(self.samples)

    def __getitem__(self, i):
        s = self.samples[i]
        ids = list(s["input_ids"])
        labels = list(s["labels"]) if "labels" in s else list(ids)
        if self.seq_length:
            width = self.seq_length + 1
            ids, labels = ids[:width], labels[:width]
            gap = width - len(ids)
            ids, labels = ids + [self.pad] * gap, labels + [IGNORE_INDEX] * gap
        out = {"input_ids": torch.tensor(ids[:-1], dtype=torch.int64), "labels": torch.tensor(labels[1:], dtype=torch.int64)}
        out["loss_mask"] = (out["labels"] != IGNORE_INDEX).float()
        for key in ("actual_seq_len", "position_ids"):
            if key in s:
                out[key] = torch.as_tensor(np.asarray(s[key]))
        return out


@MindFormerRegister.register(MindFormerModuleType.DATASET_LOADER)
class HFDataLoader:
    """Local files or directories through the Hugging Face ``datasets`` library, then data handlers.

    ``path``: a builder name (``json``, ``parquet``, ``csv``, ``text``) with ``data_files``, or a directory written by
    ``Dataset.save_to_disk``. ``handler``: list of handler configs (``AlpacaInstructDataHandler``, ``PackingHandler``
    …) applied in order to the records; without handlers the rows must already carry ``input_ids``. This is the
    reference's ``CommonDataLoader`` + ``ms_ds_convertor`` pair (``dataset/dataloader/common_dataloader.py``), with
    torch tensors at the end instead of a MindSpore dataset. No hub access: names that are not local raise.
    """

    def __new__(cls, path: str, data_files=None, split: str = "train", handler: Optional[List[dict]] = None,
                tokenizer=None, seq_length: Optional[int] = None, shuffle: bool = False, seed: int = 0,
                num_samples: Optional[int] = None, pad_token_id: int = 0, **kw):
        import datasets
        if os.path.isdir(path) and os.path.exists(os.path.join(path, "dataset_info.json")):
            ds = datasets.load_from_disk(path)
            if isinstance(ds, datasets.DatasetDict):
                ds = ds[split]
        elif path in ("json", "parquet", "csv", "text", "arrow"):
            if not data_files:
                raise ValueError(f"path={path!r} needs data_files")
            ds = datasets.load_dataset(path, data_files=data_files, split=split)
        elif os.path.exists(path):
            ext = os.path.splitext(path)[1].lstrip(".")
            builder = {"jsonl": "json", "json": "json", "parquet": "parquet", "csv": "csv", "txt": "text"}.get(ext)
            if os.path.isdir(path):
                files = list_files(path)
                ext = os.path.splitext(files[0])[1].lstrip(".")
                builder = {"jsonl": "json", "json": "json", "parquet": "parquet", "csv": "csv", "txt": "text"}[ext]
                ds = datasets.load_dataset(builder, data_files=files, split=split)
            else:
                ds = datasets.load_dataset(builder, data_files=path, split=split)
        else:
            raise FileNotFoundError(f"{path} is neither a local file / directory nor a builder name "
                                    f"(the hub cannot be reached from here)")
        if shuffle:
            ds = ds.shuffle(seed=seed)
        if num_samples:
            ds = ds.select(range(min(int(num_samples), len(ds))))
        records: List[dict] = list(ds)
        tok = _resolve_tokenizer(tokenizer) if tokenizer is not None else None
        if handler:
            from .handlers import build_data_handler
            for h in handler:
                cfg = dict(h)
                if tok is not None:
                    cfg.setdefault("tokenizer", tok)
                if seq_length:
                    cfg.setdefault("seq_length", seq_length)
                records = build_data_handler(cfg).handle(records)
        if records and "input_ids" not in records[0]:
            raise KeyError("rows carry no input_ids: add a tokenising handler")
        pid = getattr(tok, "pad_token_id", None)
        return _SampleList(records, seq_length, pad_token_id if pid is None else pid)


class MultiModalSFTDataLoader(Dataset):
    """Random-access view of a conversation-format annotation file (reference
    ``dataset/dataloader/multi_modal_dataloader.py:48``): item ``i`` is a 1-tuple holding the conversation as
    ``[[role, text], ...]``. ``map_function_kwargs``: ``data_field`` ("conversations"), ``from_keyword`` ("from"),
    ``value_keyword`` ("value"); ``read_function``: path → list of records (default: JSON / JSON lines)."""

    def __init__(self, annotation_file: str, max_length: int = 1025, read_function: Optional[Callable] = None,
                 map_function_kwargs: Optional[dict] = None, max_chunk_size: int = 1024, **kw):
        if not os.path.exists(annotation_file):
            raise FileExistsError(f"The annotation_file {annotation_file} is not exist.")
        self.max_length, self.kwargs = max_length, dict(map_function_kwargs or {})
        self.records = read_function(annotation_file) if read_function else read_records(
            annotation_file, "json" if annotation_file.endswith(".json") else None)

    def __len__(self):
        return len(self.records)

    def conversation(self, record: dict) -> List[List[str]]:
        field = self.kwargs.get("data_field", "conversations")
        fk, vk = self.kwargs.get("from_keyword", "from"), self.kwargs.get("value_keyword", "value")
        return [[m[fk], m[vk]] for m in record[field]]

    def __getitem__(self, i):
        return (self.conversation(self.records[i]),)


@MindFormerRegister.register(MindFormerModuleType.DATASET_LOADER)
class BaseMultiModalDataLoader:
    """Conversation-format annotation file → rows ``{"conversations": [[role, text], ...]}`` (reference
    ``dataset/dataloader/multi_modal_dataloader.py:30``). ``extra_kwargs`` are the arguments of
    ``MultiModalSFTDataLoader`` (``map_function_kwargs``, ``read_function``, ``max_length``)."""

    def __new__(cls, annotation_file: str, shuffle: Optional[bool] = True, extra_kwargs: Optional[dict] = None, seed: int = 0,
                **kwargs):
        extra = dict(extra_kwargs or {})
        mk = dict(extra.pop("map_function_kwargs", None) or {})
        for key in ("data_field", "from_keyword", "value_keyword"):
            if key in extra:
                mk.setdefault(key, extra.pop(key))
        source = MultiModalSFTDataLoader(annotation_file, map_function_kwargs=mk, **extra)
        rows = [{"conversations": source[i][0]} for i in range(len(source))]
        if shuffle:
            random.Random(seed).shuffle(rows)
        return _RawRecords(rows)
