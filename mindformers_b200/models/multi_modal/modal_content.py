"""Turning mixed text / image queries into model inputs.

A query is a list of parts, ``[{"image": path_or_array}, {"text": "what is this?"}]``. Each modality has a
``ModalContentBuilder``: it writes a tagged placeholder into the conversation text (``<img>…</img>``), later swaps the
tokenised placeholder for ``context_length`` copies of its pad token between a start and an end token, and records
where those pad positions are (``[batch_index, position]`` pairs) so that the model can scatter encoder outputs into
the text embeddings. ``ModalContentTransformTemplate`` drives the builders for prediction and for training
(conversations with loss on assistant turns only) and batches the results.

Reference: ``mindformers/models/multi_modal/modal_content.py`` (``ModalContentBuilder:33``,
``BaseImageContentBuilder:186``, ``ModalContentTransformTemplate:263``).
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

IGNORE_INDEX = -100


class DataRecord(dict):
    """Per-sample scratch space of the builders; keys listed in ``output_columns`` leave with the sample."""

    def put(self, key: str, value: Any, append: bool = False):
        if append:
            self.setdefault(key, []).append(value)
        else:
            self[key] = value


class ModalContentBuilder:
    """Turns the tagged content of one modality (for example ``<img>path</img>``) into model inputs: loads and
    encodes the content, pads the token sequence with ``context_length`` placeholder tokens per item and reports
    their positions (reference ``models/multi_modal/modal_content.py:37``)."""

    def __init__(self, type_: str, context_pad_token: str, context_length: int, use_custom_token_pos: bool = False,
                 start_token: Optional[str] = None, end_token: Optional[str] = None, tokenizer=None,
                 need_padding_context: bool = True, modal_content_max_size: int = 1, mode: str = "predict",
                 max_length: int = 2048):
        self.type = type_
        self.context_pad_token, self.context_length = context_pad_token, int(context_length)
        self.start_token, self.end_token = start_token, end_token
        self.tokenizer = tokenizer
        self.need_padding_context = need_padding_context
        self.modal_content_max_size = int(modal_content_max_size)
        self.mode, self.max_length = mode, max_length
        self.use_custom_token_pos = use_custom_token_pos
        self._ids_ready = False

    # ---- token ids of the markers -----------------------------------------------------------------
    def bind(self, tokenizer):
        self.tokenizer = tokenizer
        self._ids_ready = False

    def _resolve_ids(self):
        if self._ids_ready:
            return
        tid = self.tokenizer.convert_tokens_to_ids
        self.context_pad_token_id = tid(self.context_pad_token)
        self.start_token_id = tid(self.start_token) if self.start_token else None
        self.end_token_id = tid(self.end_token) if self.end_token else None
        if self.context_pad_token_id is None:
            raise ValueError(f"tokenizer has no token {self.context_pad_token!r}; add it as a special token")
        self._ids_ready = True

    # ---- text side --------------------------------------------------------------------------------
    def regular_input_for_predict(self, inputs: dict, result_recorder: DataRecord, **kwargs) -> str:
        raise NotImplementedError

    def regular_input_for_train(self, inputs, result_recorder: DataRecord, **kwargs) -> str:
        raise NotImplementedError

    @staticmethod
    def find_tag_and_extract(text: str, start_tag: str, end_tag: str, check_close: bool = True) -> List[str]:
        """Contents of every ``start_tag … end_tag`` span of ``text``, in order."""
        out, pos = [], 0
        while True:
            a = text.find(start_tag, pos)
            if a < 0:
                break
            b = text.find(end_tag, a + len(start_tag))
            if b < 0:
                if check_close:
                    raise ValueError(f"{start_tag} at {a} is never closed by {end_tag}")
                break
            out.append(text[a + len(start_tag):b])
            pos = b + len(end_tag)
        return out

    # ---- id side ----------------------------------------------------------------------------------
    def padding_context(self, input_ids: List[int], result_recorder: DataRecord, **kwargs) -> List[int]:
        """Replace every ``start … end`` span by ``start + pad × context_length + end``."""
        self._resolve_ids()
        if self.start_token_id is None or self.end_token_id is None:
            return input_ids
        out: List[int] = []
        i, n, spans = 0, len(input_ids), 0
        while i < n:
            t = input_ids[i]
            if t == self.start_token_id:
                try:
                    j = input_ids.index(self.end_token_id, i + 1)
                except ValueError as e:
                    raise ValueError(f"{self.start_token} without {self.end_token} in the tokenised text") from e
                out += [t] + [self.context_pad_token_id] * self.context_length + [self.end_token_id]
                spans += 1
                i = j + 1
            else:
                out.append(t)
                i += 1
        if spans > self.modal_content_max_size:
            raise ValueError(f"{spans} {self.type} items in one sample, at most {self.modal_content_max_size} allowed")
        return out

    def generate_context_positions(self, input_ids: Sequence[int], batch_index: int = 0,
                                   result_recorder: Optional[DataRecord] = None, **kwargs) -> np.ndarray:
        """``[n_items, context_length, 2]`` of ``(batch_index, position)``, padded to ``modal_content_max_size``."""
        self._resolve_ids()
        ids = np.asarray(input_ids)
        pos = np.where(ids == self.context_pad_token_id)[0]
        usable = (len(pos) // self.context_length) * self.context_length
        pos = pos[:usable].reshape(-1, self.context_length)
        if self.mode == "train" and len(pos) < self.modal_content_max_size:
            fill = np.tile(np.arange(self.context_length) if len(pos) == 0 else pos[-1],
                           (self.modal_content_max_size - len(pos), 1))
            pos = np.concatenate([pos, fill], axis=0) if len(pos) else fill
        batch = np.full_like(pos, batch_index)
        return np.stack([batch, pos], axis=-1).astype(np.int64)


class BaseTextContentBuilder(ModalContentBuilder):
    """The text part of a query: passes the string through."""

    def __init__(self, **kwargs):
        super().__init__("text", "", 0, need_padding_context=False, **kwargs)

    def regular_input_for_predict(self, inputs, result_recorder, **kwargs):
        return inputs["text"]

    def regular_input_for_train(self, inputs, result_recorder, **kwargs):
        return inputs if isinstance(inputs, str) else inputs["text"]

    def _resolve_ids(self):
        self._ids_ready = True


class BaseImageContentBuilder(ModalContentBuilder):
    """Images become ``<img>path</img>`` in the text; ``image_processor`` turns the loaded image into pixel values
    that are collected under ``"images"`` (padded with zeros to ``modal_content_max_size`` when training)."""

    def __init__(self, context_pad_token: str, context_length: int, image_processor=None, start_token: str = "<img>",
                 end_token: str = "</img>", image_location: str = "", **kwargs):
        super().__init__("image", context_pad_token, context_length, start_token=start_token, end_token=end_token,
                         **kwargs)
        self.image_processor = image_processor
        self.image_location = image_location

    def load_image(self, item):
        if isinstance(item, str):
            import os
            from PIL import Image
            path = item if os.path.isabs(item) or not self.image_location else os.path.join(self.image_location, item)
            return Image.open(path).convert("RGB")
        return item

    def _encode(self, item, recorder: DataRecord):
        pixels = self.image_processor(self.load_image(item)) if self.image_processor else torch.as_tensor(item)
        if pixels.dim() == 4:
            pixels = pixels[0]
        recorder.put("images", pixels, append=True)

    def regular_input_for_predict(self, inputs, result_recorder, **kwargs):
        self._encode(inputs["image"], result_recorder)
        tag = inputs["image"] if isinstance(inputs["image"], str) else "image"
        return f"{self.start_token}{tag}{self.end_token}"

    def regular_input_for_train(self, inputs, result_recorder, **kwargs):
        text = inputs if isinstance(inputs, str) else inputs.get("text", "")
        for path in self.find_tag_and_extract(text, self.start_token, self.end_token):
            self._encode(path, result_recorder)
        return text


class ModalContentTransformTemplate:
    """Builds ``input_ids`` (+ ``labels``), modal tensors and context positions for one sample, and batches samples.

    Subclasses adapt ``build_conversation_input_text`` (prompt format) and may add builders. ``output_columns`` names
    the keys returned by ``batch``; the default is ``input_ids``, ``images``, ``image_context_pos`` (+ ``labels``
    in train mode).
    """

    def __init__(self, tokenizer=None, modal_builders: Optional[Dict[str, ModalContentBuilder]] = None,
                 output_columns: Optional[List[str]] = None, mode: str = "predict", max_length: int = 2048,
                 ignore_token_id: int = IGNORE_INDEX, user_role: str = "user", assistant_role: str = "assistant",
                 user_prompt: str = "", assistant_prompt: str = "", **kwargs):
        self.tokenizer, self.mode, self.max_length = tokenizer, mode, int(max_length)
        self.ignore_token_id = ignore_token_id
        self.user_role, self.assistant_role = user_role, assistant_role
        self.user_prompt, self.assistant_prompt = user_prompt, assistant_prompt
        self.modal_builders: Dict[str, ModalContentBuilder] = {"text": BaseTextContentBuilder()}
        self.modal_builders.update(modal_builders or {})
        for b in self.modal_builders.values():
            b.mode, b.max_length = mode, self.max_length
            if tokenizer is not None:
                b.bind(tokenizer)
        self.output_columns = output_columns or (["input_ids", "images", "image_context_pos"]
                                                 + (["labels"] if mode == "train" else []))

    @property
    def supported_modal(self) -> List[str]:
        return list(self.modal_builders)

    def check_modal_builder_tokens(self, tokenizer):
        for b in self.modal_builders.values():
            b.bind(tokenizer)
            b._resolve_ids()

    # ---- text -------------------------------------------------------------------------------------
    def build_conversation_input_text(self, raw_inputs, result_recorder: DataRecord) -> str:
        if self.mode == "predict":
            return self.user_prompt + "".join(raw_inputs) + self.assistant_prompt
        return "".join(text for _, text in raw_inputs)

    def process_predict_query(self, query_ele_list: List[dict], result_recorder: DataRecord) -> str:
        parts = []
        for ele in query_ele_list:
            kind = next((k for k in ele if k in self.modal_builders), None)
            if kind is None:
                raise KeyError(f"query part {ele!r}: supported modalities are {self.supported_modal}")
            parts.append(self.modal_builders[kind].regular_input_for_predict(ele, result_recorder))
        return self.build_conversation_input_text(parts, result_recorder)

    def process_train_item(self, conversation_list: List[Tuple[str, str]], result_recorder: DataRecord):
        """``[(role, text), …]`` → the same with every builder having seen (and encoded) its tagged content."""
        out = []
        for role, text in conversation_list:
            for name, b in self.modal_builders.items():
                if name != "text":
                    text = b.regular_input_for_train(text, result_recorder)
            out.append((role, text))
        return out

    # ---- ids --------------------------------------------------------------------------------------
    def build_modal_context(self, input_ids: List[int], result_recorder: DataRecord, **kwargs) -> List[int]:
        for b in self.modal_builders.values():
            if b.need_padding_context:
                input_ids = b.padding_context(input_ids, result_recorder, **kwargs)
        return input_ids

    def build_labels(self, turns: List[Tuple[str, List[int]]], result_recorder: DataRecord) -> List[int]:
        labels: List[int] = []
        for role, ids in turns:
            labels += list(ids) if role == self.assistant_role else [self.ignore_token_id] * len(ids)
        return labels

    def generate_modal_context_positions(self, input_ids, batch_index: int = 0,
                                         result_recorder: Optional[DataRecord] = None) -> Dict[str, np.ndarray]:
        return {f"{name}_context_pos": b.generate_context_positions(input_ids, batch_index, result_recorder)
                for name, b in self.modal_builders.items() if b.need_padding_context}

    def encode_predict(self, query_ele_list: List[dict], batch_index: int = 0) -> DataRecord:
        rec = DataRecord()
        text = self.process_predict_query(query_ele_list, rec)
        ids = list(self.tokenizer.encode(text, add_special_tokens=True))
        ids = self.build_modal_context(ids, rec)
        rec.put("raw_query", text)
        rec.put("input_ids", ids)
        rec.update(self.generate_modal_context_positions(ids, batch_index, rec))
        return rec

    def encode_train(self, conversation_list: List[Tuple[str, str]], batch_index: int = 0) -> DataRecord:
        rec = DataRecord()
        conv = self.process_train_item(conversation_list, rec)
        turns = []
        for role, text in conv:
            prefix = self.user_prompt if role == self.user_role else self.assistant_prompt
            ids = list(self.tokenizer.encode(prefix + text, add_special_tokens=False))
            if role == self.assistant_role and self.tokenizer.eos_token_id is not None:
                ids.append(self.tokenizer.eos_token_id)
            turns.append((role, self.build_modal_context(ids, rec)))
        ids = [t for _, part in turns for t in part]
        labels = self.build_labels(turns, rec)
        ids, labels = ids[:self.max_length], labels[:self.max_length]
        gap = self.max_length - len(ids)
        pad = self.tokenizer.pad_token_id if self.tokenizer.pad_token_id is not None else 0
        ids, labels = ids + [pad] * gap, labels + [self.ignore_token_id] * gap
        rec.put("input_ids", ids[:-1])
        rec.put("labels", labels[1:])
        rec.update(self.generate_modal_context_positions(ids[:-1], batch_index, rec))
        return rec

    # ---- batches ----------------------------------------------------------------------------------
    def batch_input_ids(self, input_ids_list: List[List[int]], max_length: Optional[int] = None) -> torch.Tensor:
        width = max_length or max(len(x) for x in input_ids_list)
        pad = self.tokenizer.pad_token_id if self.tokenizer.pad_token_id is not None else 0
        rows = [list(x)[:width] + [pad] * (width - len(x)) for x in input_ids_list]
        return torch.tensor(rows, dtype=torch.int64)

    def batch(self, data_list: List[DataRecord], token_padding_length: Optional[int] = None) -> Dict[str, Any]:
        out: Dict[str, Any] = {}
        for col in self.output_columns:
            vals = [d[col] for d in data_list if col in d]
            if not vals:
                continue
            if col in ("input_ids", "labels"):
                if col == "labels":
                    width = token_padding_length or max(len(v) for v in vals)
                    out[col] = torch.tensor([list(v) + [self.ignore_token_id] * (width - len(v)) for v in vals])
                else:
                    out[col] = self.batch_input_ids(vals, token_padding_length)
            elif col.endswith("_context_pos"):
                out[col] = torch.from_numpy(np.concatenate([v for v in vals if len(v)], axis=0)) if any(
                    len(v) for v in vals) else torch.zeros(0, 0, 2, dtype=torch.int64)
            else:
                flat = [t for v in vals for t in (v if isinstance(v, list) else [v])]
                out[col] = torch.stack([torch.as_tensor(t) for t in flat])
        return out

    def post_process(self, output_ids, **kwargs) -> List[str]:
        return self.tokenizer.batch_decode(output_ids, skip_special_tokens=kwargs.get("skip_special_tokens", True))
