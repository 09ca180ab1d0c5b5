"""Datasets and loaders registered for the YAML ``train_dataset`` / ``train_dataset_task`` sections.

Reference: ``dataset/causal_language_model_dataset.py`` (:188-377: sharding by data-parallel rank, batching with
drop-remainder, EOD-reset maps, int32 cast), ``dataset/dataloader/blended_megatron_dataloader.py`` (:41-306: only
the first tensor-parallel rank of the first/last pipeline stage reads real data, others get fake samples),
``dataset/dataloader/*`` (common / SFT / indexed loaders), ``dataset/base_dataset.py`` (shard id / num shards).
Here everything is a ``torch.utils.data.DataLoader`` with a resumable sampler.
"""
from __future__ import annotations

import json
import os
from typing import Callable, Dict, Iterator, List, Optional

import numpy as np
import torch
from torch.utils.data import DataLoader, Dataset, Sampler

from ..parallel import parallel_state as ps
from ..tools.register import MindFormerModuleType, MindFormerRegister
from .gpt_dataset import BlendedMegatronDatasetBuilder, GPTDataset, GPTDatasetConfig, MockGPTDataset


class ResumableShardSampler(Sampler):
    """Deterministic shuffled shard of the index space with a fast-forward for resume (``set_init_step``)."""

    def __init__(self, size: int, num_shards: int = 1, shard_id: int = 0, shuffle: bool = False, seed: int = 0,
                 drop_last: bool = True):
        self.size, self.num_shards, self.shard_id = size, num_shards, shard_id
        self.shuffle, self.seed, self.drop_last = shuffle, seed, drop_last
        self.epoch, self.skip = 0, 0

    def set_epoch(self, epoch: int):
        self.epoch = epoch

    def set_skip(self, num_samples: int):
        self.skip = num_samples

    def __len__(self):
        return self.size // self.num_shards

    def __iter__(self) -> Iterator[int]:
        if self.shuffle:
            order = np.random.RandomState(self.seed + self.epoch).permutation(self.size)
        else:
            order = np.arange(self.size)
        # strided shards (sample i of the order goes to shard i % num_shards, as MindSpore's distributed sampler
        # does): the samples of global step s are order[s*G : (s+1)*G] for every data-parallel size, so a run that
        # resumes under another layout continues with exactly the data the old layout would have seen
        per = self.size // self.num_shards
        mine = order[self.shard_id::self.num_shards][:per]
        start, self.skip = self.skip, 0
        return iter(mine[start:].tolist())


def collate(batch: List[Dict[str, torch.Tensor]]) -> Dict[str, torch.Tensor]:
    return {k: torch.stack([b[k] for b in batch]) for k in batch[0] if isinstance(batch[0][k], torch.Tensor)}


def data_shard_info():
    """(num_shards, shard_id) of this rank = its data-parallel coordinates."""
    return ps.get_data_parallel_world_size(), ps.get_data_parallel_rank()


class _TokenFileDataset(Dataset):
    """Pre-tokenised samples from a ``.npy`` / ``.jsonl`` file with an ``input_ids`` column."""

    def __init__(self, path: str, seq_length: int, column: str = "input_ids", pad_token_id: int = 0):
        self.seq_length, self.pad = seq_length, pad_token_id
        if path.endswith(".npy"):
            self.rows = np.load(path, mmap_mode="r")
        else:
            self.rows = []
            with open(path) as f:
                for line in f:
                    if line.strip():
                        self.rows.append(json.loads(line)[column])

    def __len__(self):
        return len(self.rows)

    def __getitem__(self, i):
        ids = np.asarray(self.rows[i], dtype=np.int64)[: self.seq_length + 1]
        if ids.shape[0] < self.seq_length + 1:
            ids = np.concatenate((ids, np.full(self.seq_length + 1 - ids.shape[0], self.pad, dtype=np.int64)))
        t = torch.from_numpy(ids.copy())
        return {"input_ids": t[:-1], "labels": t[1:], "loss_mask": (t[1:] != self.pad).float()}


@MindFormerRegister.register(MindFormerModuleType.DATASET_LOADER)
class BlendedMegatronDatasetDataLoader:
    """Factory for Megatron-format data (or synthetic data when ``mock: True`` / no ``data_path``)."""

    def __new__(cls, datasets_type: str = "GPTDataset", sizes=(1000, 0, 0), config: Optional[dict] = None,
                shuffle: bool = False, **kwargs):
        cfg = dict(config or {})
        data_path = cfg.pop("data_path", None)
        blend = None
        if data_path:
            prefixes, weights = [], []
            items = list(data_path)
            if len(items) > 1 and _is_number(items[0]):
                for w, p in zip(items[0::2], items[1::2]):
                    weights.append(float(w))
                    prefixes.append(p)
            else:
                prefixes = items
            blend = (prefixes, weights or None)
        known = {f.name for f in GPTDatasetConfig.__dataclass_fields__.values()}
        gcfg = GPTDatasetConfig(sequence_length=cfg.pop("seq_length", cfg.pop("sequence_length", 4096)), blend=blend,
                                **{k: v for k, v in cfg.items() if k in known})
        if blend is None:
            gcfg.mock = True
        # only the ranks that feed the model read files; the others get synthetic placeholders
        reader = ps.get_tensor_model_parallel_rank() == 0 and (ps.is_pipeline_first_stage(True) or ps.is_pipeline_last_stage(True))
        if not reader:
            gcfg.mock = True
        return BlendedMegatronDatasetBuilder(GPTDataset, list(sizes), gcfg).build()[0]


def _is_number(x) -> bool:
    try:
        float(x)
        return True
    except (TypeError, ValueError):
        return False


@MindFormerRegister.register(MindFormerModuleType.DATASET_LOADER)
class IndexedDataLoader:
    """Samples of ``seq_length + 1`` tokens cut from one ``.bin`` / ``.idx`` prefix (reference
    ``dataset/dataloader/indexed_dataset.py``)."""

    def __new__(cls, path_prefix: str, seq_length: int = 4096, num_samples: Optional[int] = None, seed: int = 1234, **kw):
        from .indexed_dataset import IndexedDataset
        indexed = IndexedDataset(path_prefix)
        gcfg = GPTDatasetConfig(sequence_length=seq_length, random_seed=seed)
        return GPTDataset(indexed, path_prefix, np.arange(len(indexed), dtype=np.int32), num_samples, "train", gcfg)


@MindFormerRegister.register(MindFormerModuleType.DATASET_LOADER)
class CommonDataLoader:
    """Pre-tokenised ``.jsonl`` / ``.npy`` files (the HF-datasets loader of the reference reduced to local files)."""

    def __new__(cls, path: str = None, dataset_dir: str = None, seq_length: int = 4096, input_columns=("input_ids",),
                pad_token_id: int = 0, **kw):
        return _TokenFileDataset(path or dataset_dir, seq_length, input_columns[0], pad_token_id)


@MindFormerRegister.register(MindFormerModuleType.DATASET_LOADER)
class MockDataLoader:
    """Uniform random token ids of the configured shape: data for benchmarks and smoke runs."""

    def __new__(cls, seq_length: int = 4096, vocab_size: int = 32000, num_samples: int = 1 << 20, seed: int = 1234, **kw):
        return MockGPTDataset(num_samples, GPTDatasetConfig(sequence_length=seq_length, random_seed=seed,
                                                            vocab_size=vocab_size), vocab_size)


def build_dataset_loader(config: dict, default_args: Optional[dict] = None):
    return MindFormerRegister.get_instance_from_cfg(dict(config), MindFormerModuleType.DATASET_LOADER,
                                                    default_args=default_args)


@MindFormerRegister.register(MindFormerModuleType.DATASET)
class CausalLanguageModelDataset:
    """``CausalLanguageModelDataset(dataset_config)`` → batched iterator of dicts of tensors.

    Keys used from the configuration: ``data_loader`` (registry entry), ``batch_size``, ``drop_remainder``,
    ``shuffle``, ``seed``, ``num_parallel_workers``, ``input_columns``, ``pin_memory``.
    """

    def __new__(cls, dataset_config: Optional[dict] = None, **kwargs):
        cfg = dict(dataset_config or {})
        cfg.update(kwargs)
        loader_cfg = cfg.get("data_loader") or {"type": "MockDataLoader"}
        dataset = build_dataset_loader(loader_cfg) if isinstance(loader_cfg, dict) else loader_cfg
        shards, shard_id = data_shard_info()
        sampler = ResumableShardSampler(len(dataset), shards, shard_id, bool(cfg.get("shuffle", False)),
                                        int(cfg.get("seed", 0) or 0))
        loader = DataLoader(dataset, batch_size=int(cfg.get("batch_size", 1)), sampler=sampler,
                            drop_last=bool(cfg.get("drop_remainder", True)), collate_fn=collate,
                            num_workers=int(cfg.get("num_parallel_workers", 0) or 0),
                            pin_memory=bool(cfg.get("pin_memory", torch.cuda.is_available())))
        loader.shard_sampler = sampler
        loader.set_init_step = lambda steps, bs=int(cfg.get("batch_size", 1)): sampler.set_skip(steps * bs)
        if cfg.get("token_monitor"):
            loader.collate_fn = TokenMonitor(collate, **dict(cfg.get("token_monitor_config") or {}))
            loader.token_monitor = loader.collate_fn
        return loader


class TokenMonitor:
    """Counts how often every token id is fed to the model (reference ``causal_language_model_dataset.py:448``: the
    token histogram of the training data, for spotting a tokenizer / corpus mismatch or a dominating token).

    Wraps the collate function, so it sees exactly the batches that the training loop gets (with ``num_workers > 0``
    each worker counts its own share). ``summary(top_k)`` gives totals and the most frequent ids; every
    ``dump_interval`` batches the histogram is written to ``<save_dir>/token_counts_rank<r>.npy``."""

    def __init__(self, collate_fn, vocab_size: Optional[int] = None, column: str = "input_ids", pad_token_id=None,
                 dump_interval: int = 0, save_dir: Optional[str] = None):
        self.collate_fn, self.column, self.pad = collate_fn, column, pad_token_id
        self.counts = torch.zeros(int(vocab_size or 0), dtype=torch.int64)
        self.batches, self.dump_interval, self.save_dir = 0, int(dump_interval or 0), save_dir

    def __call__(self, items):
        batch = self.collate_fn(items)
        ids = batch.get(self.column) if isinstance(batch, dict) else None
        if ids is not None:
            flat = ids.reshape(-1).to(torch.int64)
            flat = flat[flat >= 0]
            if self.pad is not None:
                flat = flat[flat != self.pad]
            if flat.numel():
                c = torch.bincount(flat, minlength=self.counts.numel())
                if c.numel() > self.counts.numel():
                    self.counts = torch.nn.functional.pad(self.counts, (0, c.numel() - self.counts.numel()))
                self.counts[: c.numel()] += c
            self.batches += 1
            if self.dump_interval and self.batches % self.dump_interval == 0:
                self.dump()
        return batch

    def summary(self, top_k: int = 10) -> dict:
        total = int(self.counts.sum())
        k = min(top_k, int((self.counts > 0).sum()))
        vals, idx = torch.topk(self.counts, k) if k else (torch.zeros(0), torch.zeros(0))
        return {"batches": self.batches, "tokens": total, "distinct": int((self.counts > 0).sum()),
                "top": [(int(i), int(v), (int(v) / total if total else 0.0)) for i, v in zip(idx.tolist(), vals.tolist())]}

    def dump(self) -> Optional[str]:
        import numpy as np
        from ..tools.utils import get_output_root_path, get_real_rank
        root = self.save_dir or os.path.join(get_output_root_path(), "token_monitor")
        os.makedirs(root, exist_ok=True)
        path = os.path.join(root, f"token_counts_rank{get_real_rank()}.npy")
        np.save(path, self.counts.numpy())
        return path


def _batched(dataset, cfg: dict, collate_fn=collate):
    shards, shard_id = data_shard_info()
    custom = (cfg.get("data_loader") or {}).get("sampler") if isinstance(cfg.get("data_loader"), dict) else None
    custom = custom or cfg.get("sampler")
    if custom:
        # ``sampler: {type: ..., ...}`` in the dataset section (reference dataset/sampler/build_sampler.py): the named
        # sampler replaces the resumable shard sampler; samplers that ask for it get the dataset size and the shard
        from .sampler import build_sampler
        import inspect
        spec = dict(custom)
        from ..tools.register import MindFormerModuleType, MindFormerRegister
        params = inspect.signature(MindFormerRegister.get_cls(MindFormerModuleType.DATASET_SAMPLER, spec["type"]).__init__).parameters
        for key, val in (("dataset_size", len(dataset)), ("num_shards", shards), ("shard_id", shard_id)):
            if key in params and key not in spec:
                spec[key] = val
        sampler = build_sampler(spec)
    else:
        sampler = ResumableShardSampler(len(dataset), shards, shard_id, bool(cfg.get("shuffle", False)),
                                        int(cfg.get("seed", 0) or 0))
    bs = int(cfg.get("batch_size", 1))
    loader = DataLoader(dataset, batch_size=bs, sampler=sampler, drop_last=bool(cfg.get("drop_remainder", True)),
                        collate_fn=collate_fn, num_workers=int(cfg.get("num_parallel_workers", 0) or 0),
                        pin_memory=bool(cfg.get("pin_memory", torch.cuda.is_available())))
    loader.shard_sampler = sampler
    loader.set_init_step = (lambda steps: sampler.set_skip(steps * bs)) if hasattr(sampler, "set_skip") else (lambda steps: None)
    return loader


def _task_tokenizer(cfg: dict):
    tok = cfg.get("tokenizer")
    if isinstance(tok, (dict, str)):
        from ..models.tokenization import build_tokenizer
        tok = build_tokenizer({"pretrained_model_dir": tok} if isinstance(tok, str) else tok)
    if tok is None:
        raise ValueError("dataset_config.tokenizer is required")
    return tok


class _KeyWordGenRows(Dataset):
    """Prompt/answer rows → model inputs (reference ``keyword_gen_dataset.py`` train / eval functions)."""

    def __init__(self, rows, tokenizer, cfg: dict):
        self.rows, self.tok = rows, tokenizer
        self.src_len = int(cfg.get("max_source_length", 64))
        self.tgt_len = int(cfg.get("max_target_length", 64))
        self.phase = cfg.get("phase", "train")
        self.ignore_pad = bool(cfg.get("ignore_pad_token_for_loss", True))
        self.prompt_col = cfg.get("prompt_column", "prompt")
        self.answer_col = cfg.get("response_column", cfg.get("answer_column", "answer"))
        pid = getattr(tokenizer, "pad_token_id", None)
        self.pad_id = 0 if pid is None else pid

    def __len__(self):
        return len(self.rows)

    def _enc(self, text, limit):
        return list(self.tok.encode(str(text), add_special_tokens=False))[:limit]

    def __getitem__(self, i):
        r = self.rows[i]
        prefix = list(self.tok.build_inputs_with_special_tokens([])) if hasattr(
            self.tok, "build_inputs_with_special_tokens") else []
        eos = self.tok.eos_token_id
        prompt = prefix + self._enc(r[self.prompt_col], self.src_len - len(prefix))
        answer = self._enc(r[self.answer_col], self.tgt_len - 1) + [eos]
        if self.phase == "train":
            width = self.src_len + self.tgt_len
            ids = prompt + answer
            labels = [-100] * len(prompt) + answer
            gap = width - len(ids)
            ids = ids + [self.pad_id] * gap
            labels = labels + [-100 if self.ignore_pad else self.pad_id] * gap
            # position t predicts token t+1
            return {"input_ids": torch.tensor(ids[:-1]), "labels": torch.tensor(labels[1:])}
        ids = [self.pad_id] * (self.src_len - len(prompt)) + prompt            # left padding for generation
        lab = answer + [self.pad_id] * (self.tgt_len - len(answer))
        return {"input_ids": torch.tensor(ids), "labels": torch.tensor(lab)}


@MindFormerRegister.register(MindFormerModuleType.DATASET)
class KeyWordGenDataset:
    """Keyword → text generation data (ADGEN style). ``dataset_config`` keys: ``data_loader`` (rows with
    ``prompt_column`` / ``response_column``), ``tokenizer``, ``max_source_length``, ``max_target_length``,
    ``ignore_pad_token_for_loss``, ``phase`` (``train`` rows are prompt+answer with prompt labels ignored; ``eval``
    rows are the left-padded prompt and the answer), and the batching keys of ``CausalLanguageModelDataset``."""

    def __new__(cls, dataset_config: Optional[dict] = None, **kwargs):
        cfg = dict(dataset_config or {})
        cfg.update(kwargs)
        loader_cfg = cfg["data_loader"]
        if isinstance(loader_cfg, dict):
            cfg.setdefault("phase", loader_cfg.get("phase", "train"))
            rows = build_dataset_loader(loader_cfg)
        else:
            rows = loader_cfg
        return _batched(_KeyWordGenRows(rows, _task_tokenizer(cfg), cfg), cfg)


TOOL_DEFINITION_PREFIX = "Answer the following questions as best as you can. You have access to the following tools:\n"
FUNCTION_CALL_NAME = "tool_call"


def format_function_call(name: str, parameters: dict) -> str:
    """``name(arg='value', …)`` as python source."""
    return f"{name}(" + ", ".join(f"{k}={v!r}" for k, v in parameters.items()) + ")"


class _MultiTurnRows(Dataset):
    """Conversations → ``input_ids`` / ``labels`` with loss on assistant turns only
    (reference ``multi_turn_dataset.py:200-268``)."""

    def __init__(self, rows, tokenizer, cfg: dict):
        self.rows, self.tok = rows, tokenizer
        self.max_len = int(cfg.get("max_seq_length", 2048))
        self.conv_key = cfg.get("conversation_key", "conversations")
        self.tool_key = cfg.get("tool_key", "tools")
        pid = getattr(tokenizer, "pad_token_id", None)
        self.pad_id = 0 if pid is None else pid

    def __len__(self):
        return len(self.rows)

    def _message(self, role, metadata, content):
        if hasattr(self.tok, "build_single_message"):
            return list(self.tok.build_single_message(role, metadata, content))
        return list(self.tok.encode(f"<|{role}|>{metadata}\n{content}", add_special_tokens=False))

    def format(self, item):
        prefix = list(self.tok.get_prefix_tokens()) if hasattr(self.tok, "get_prefix_tokens") else []
        tokens, mask = list(prefix), [0] * len(prefix)

        def put(ids, loss):
            tokens.extend(ids)
            mask.extend([int(bool(loss))] * len(ids))

        conv = [dict(c) for c in item[self.conv_key]]
        if self.tool_key in item and item[self.tool_key]:
            import json
            conv.insert(0, {"role": "system",
                            "content": TOOL_DEFINITION_PREFIX + json.dumps(item[self.tool_key], ensure_ascii=False)})
        for c in conv:
            loss = c.get("loss", True) and c["role"] not in ("system", "user")
            if c["role"] == "tool":
                call = "```python\n" + format_function_call(FUNCTION_CALL_NAME, c.get("parameters", {})) + "\n```"
                put(self._message("assistant", c.get("name", ""), call), loss)
                obs = c.get("observation")
                if not isinstance(obs, str):
                    import json
                    obs = json.dumps(obs, ensure_ascii=False)
                put(self._message("observation", "", obs), False)
            else:
                put(self._message(c["role"], "", c["content"]), loss)
        put([self.tok.eos_token_id], False)
        return tokens, mask

    def __getitem__(self, i):
        tokens, mask = self.format(self.rows[i])
        # a token carries loss if it belongs to an assistant turn; the label of position t is token t+1
        labels = [(t if m else -100) for t, m in zip(tokens, [0] + mask[:-1])]
        ids = tokens[:self.max_len]
        labels = labels[1:self.max_len]
        ids = ids + [self.pad_id] * (self.max_len - len(ids))
        labels = labels + [-100] * (self.max_len - len(labels))
        return {"input_ids": torch.tensor(ids[:-1]), "labels": torch.tensor(labels[:self.max_len - 1])}


@MindFormerRegister.register(MindFormerModuleType.DATASET)
class MultiTurnDataset:
    """Multi-turn (tool) chat data. ``dataset_config`` keys: ``data_loader`` (rows with ``conversations`` and
    optionally ``tools``), ``tokenizer`` (one with ``build_single_message`` formats turns with its role tokens),
    ``max_seq_length``, plus the batching keys of ``CausalLanguageModelDataset``."""

    def __new__(cls, dataset_config: Optional[dict] = None, **kwargs):
        cfg = dict(dataset_config or {})
        cfg.update(kwargs)
        loader_cfg = cfg["data_loader"]
        rows = build_dataset_loader(loader_cfg) if isinstance(loader_cfg, dict) else loader_cfg
        return _batched(_MultiTurnRows(rows, _task_tokenizer(cfg), cfg), cfg)


@MindFormerRegister.register(MindFormerModuleType.DATASET)
class GeneralDataset(CausalLanguageModelDataset):
    """Any map-style dataset object passed as ``data_loader``."""


def build_dataset(config: Optional[dict] = None, default_args: Optional[dict] = None, **kwargs):
    """``config = {"type": "CausalLanguageModelDataset", "dataset_config": {...}}`` (the YAML ``*_dataset_task``)."""
    if config is None:
        return None
    cfg = dict(config)
    cfg.update(kwargs)
    return MindFormerRegister.get_instance_from_cfg(cfg, MindFormerModuleType.DATASET, default_args=default_args)
