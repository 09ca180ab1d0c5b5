"""Supervised fine-tuning dataset for models that read images (or other modalities) next to text.

Reference: ``mindformers/dataset/modal_to_text_sft_dataset.py`` (``ModalToTextSFTDataset``: annotation records with
conversations and modality files → ``input_ids``, ``labels``, the modality tensors and the positions where their
context tokens sit) on top of ``models/multi_modal`` (``ModalContentTransformTemplate.encode_train`` / ``batch``).

An annotation file is a JSON list (or JSON lines) of ``{"conversations": [[role, text], ...]}`` or LLaVA-style
``{"image": ..., "conversations": [{"from": "human", "value": ...}, ...]}``; tagged content such as
``<img>path</img>`` is loaded and encoded by the template's modality builders.
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, List, Optional

import torch
from torch.utils.data import DataLoader, Dataset

from ..tools.register import MindFormerModuleType, MindFormerRegister


def _read_annotations(path: str) -> List[dict]:
    with open(path) as f:
        head = f.read(1)
        f.seek(0)
        if head == "[":
            return json.load(f)
        return [json.loads(line) for line in f if line.strip()]


class _ModalRows(Dataset):
    def __init__(self, records: List[dict], template, image_dir: str = "", image_tag=("<img>", "</img>"),
                 user_role: str = "user", assistant_role: str = "assistant"):
        self.records, self.template, self.image_dir, self.tag = records, template, image_dir, image_tag
        self.user_role, self.assistant_role = user_role, assistant_role

    def __len__(self):
        return len(self.records)

    def conversation(self, rec: dict):
        conv = []
        turns = rec.get("conversations") or []
        for i, turn in enumerate(turns):
            if isinstance(turn, dict):                      # LLaVA style
                role = self.user_role if turn.get("from") in ("human", "user") else self.assistant_role
                text = turn.get("value", "")
                if rec.get("image") and "<image>" in text:
                    path = os.path.join(self.image_dir, rec["image"]) if self.image_dir else rec["image"]
                    text = text.replace("<image>", f"{self.tag[0]}{path}{self.tag[1]}")
            else:
                role, text = turn
            conv.append((role, text))
        return conv

    def __getitem__(self, i):
        return self.template.encode_train(self.conversation(self.records[i]), batch_index=0)


@MindFormerRegister.register(MindFormerModuleType.DATASET)
class ModalToTextSFTDataset:
    """``ModalToTextSFTDataset(dataset_config)`` → an iterable of batches ``{"input_ids", "labels", <modal tensors>,
    "<modal>_context_pos"}``. ``dataset_config``: ``annotation_file`` (or ``data_loader.annotation_file``),
    ``modal_content_transform_template`` (an object or a registry config), ``image_dir``, ``batch_size``,
    ``shuffle``, ``drop_remainder``, ``max_length``."""

    def __new__(cls, dataset_config: Optional[dict] = None, **kwargs):
        cfg = dict(dataset_config or {})
        cfg.update(kwargs)
        loader_cfg = dict(cfg.get("data_loader") or {})
        ann = cfg.get("annotation_file") or loader_cfg.get("annotation_file")
        if not ann:
            raise ValueError("ModalToTextSFTDataset needs annotation_file")
        template = cfg.get("modal_content_transform_template") or cfg.get("template")
        if isinstance(template, dict):
            from ..tools.register import MindFormerRegister as R
            template = R.get_instance_from_cfg(template, MindFormerModuleType.TRANSFORMS)
        if template is None:
            raise ValueError("ModalToTextSFTDataset needs modal_content_transform_template")
        tok = cfg.get("tokenizer")
        if tok is not None and getattr(template, "tokenizer", None) is None:
            template.tokenizer = tok
            for b in template.modal_builders.values():
                b.bind(tok)
        if cfg.get("max_length"):
            template.max_length = int(cfg["max_length"])
        rows = _ModalRows(_read_annotations(ann), template, cfg.get("image_dir", loader_cfg.get("image_dir", "")))
        pad_to = cfg.get("token_padding_length")

        def collate(items: List[Any]) -> Dict[str, torch.Tensor]:
            # context positions index into the batch: row b of the batch is item b
            for b, rec in enumerate(items):
                for k in list(rec):
                    if k.endswith("_context_pos") and len(rec[k]):
                        rec[k] = rec[k].copy()
                        rec[k][..., 0] = b
            return template.batch(items, pad_to)

        return DataLoader(rows, batch_size=int(cfg.get("batch_size", 1)), shuffle=bool(cfg.get("shuffle", False)),
                          drop_last=bool(cfg.get("drop_remainder", True)), collate_fn=collate,
                          num_workers=int(cfg.get("num_parallel_workers", 0) or 0))
