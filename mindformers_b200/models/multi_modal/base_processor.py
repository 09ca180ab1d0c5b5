"""Image pre-processing and the processor object that multimodal pipelines call.

Reference: ``mindformers/models/multi_modal/base_multi_modal_processor.py`` (``BaseImageToTextImageProcessor:55``,
``BaseXModalToTextTransform:117``, ``BaseXModalToTextProcessor:252``) and ``models/image_processing_utils.py``
(``BaseImageProcessor``).
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Sequence, Union

import numpy as np
import torch
import torch.nn.functional as F

from ...tools.register import MindFormerModuleType, MindFormerRegister
from .modal_content import DataRecord, ModalContentTransformTemplate

OPENAI_CLIP_MEAN = (0.48145466, 0.4578275, 0.40821073)
OPENAI_CLIP_STD = (0.26862954, 0.26130258, 0.27577711)


class BaseImageProcessor:
    """Callable ``images → tensor``; subclasses implement ``preprocess``."""

    def __init__(self, **kwargs):
        self.config = dict(kwargs)

    def __call__(self, images, **kwargs):
        return self.preprocess(images, **kwargs)

    def preprocess(self, images, **kwargs):
        raise NotImplementedError


@MindFormerRegister.register(MindFormerModuleType.PROCESSOR)
class BaseImageToTextImageProcessor(BaseImageProcessor):
    """PIL image / ``HWC`` uint8 array / ``CHW`` float tensor (or a list of them) → ``[N, 3, size, size]`` float
    tensor: bicubic resize, scale to ``[0, 1]``, normalise with ``mean`` / ``std``."""

    def __init__(self, image_size: int = 224, interpolation: str = "bicubic", mean: Sequence[float] = OPENAI_CLIP_MEAN,
                 std: Sequence[float] = OPENAI_CLIP_STD, is_hwc: bool = False, **kwargs):
        super().__init__(image_size=image_size, interpolation=interpolation, mean=mean, std=std)
        self.image_size = int(image_size)
        self.interpolation = interpolation
        self.mean = torch.tensor(mean, dtype=torch.float32).view(1, 3, 1, 1)
        self.std = torch.tensor(std, dtype=torch.float32).view(1, 3, 1, 1)

    def _to_chw(self, image) -> torch.Tensor:
        if isinstance(image, torch.Tensor):
            t = image.float()
            if t.dim() == 3 and t.shape[-1] == 3 and t.shape[0] != 3:
                t = t.permute(2, 0, 1)
            return t / 255.0 if t.max() > 1.5 else t
        arr = np.asarray(image)
        if arr.ndim == 2:
            arr = np.stack([arr] * 3, axis=-1)
        if arr.ndim != 3 or arr.shape[-1] not in (3, 4):
            raise ValueError(f"expected an HWC image, got shape {arr.shape}")
        t = torch.from_numpy(np.array(arr[..., :3], copy=True)).permute(2, 0, 1).float()
        return t / 255.0 if arr.dtype == np.uint8 or t.max() > 1.5 else t

    def preprocess(self, images, **kwargs) -> torch.Tensor:
        if isinstance(images, torch.Tensor) and images.dim() == 4:
            items = list(images)
        elif isinstance(images, (list, tuple)):
            items = list(images)
        else:
            items = [images]
        out = []
        for im in items:
            t = self._to_chw(im).unsqueeze(0)
            if t.shape[-2:] != (self.image_size, self.image_size):
                t = F.interpolate(t, size=(self.image_size, self.image_size), mode=self.interpolation,
                                  align_corners=False, antialias=self.interpolation in ("bilinear", "bicubic"))
            out.append(((t.clamp(0, 1) - self.mean) / self.std)[0])
        return torch.stack(out)


class BaseXModalToTextTransform:
    """Dataset-side transform: conversations → one training sample (``input_ids``, ``labels``, modal tensors)."""

    def __init__(self, tokenizer, model_transform_template: ModalContentTransformTemplate, max_length: int = 2048,
                 **kwargs):
        self.tokenizer, self.template, self.max_length = tokenizer, model_transform_template, max_length
        self.template.tokenizer = tokenizer
        self.template.check_modal_builder_tokens(tokenizer)

    @staticmethod
    def process_conversation(conversations) -> List[tuple]:
        """``[{"from"|"role": …, "value"|"content": …}, …]`` or ``[[role, text], …]`` → ``[(role, text), …]``."""
        out = []
        for c in conversations:
            if isinstance(c, dict):
                out.append((c.get("from", c.get("role")), c.get("value", c.get("content", ""))))
            else:
                out.append((c[0], c[1]))
        return out

    def __call__(self, conversations, batch_index: int = 0, **kwargs) -> DataRecord:
        mode = self.template.mode
        if mode == "train":
            return self.template.encode_train(self.process_conversation(conversations), batch_index)
        return self.template.encode_predict(conversations, batch_index)


@MindFormerRegister.register(MindFormerModuleType.PROCESSOR)
class BaseXModalToTextProcessor:
    """``processor(query_list)`` → batched model inputs for ``generate``; ``post_process`` decodes output ids.

    ``query_list`` is one query (list of parts) or a batch of queries.
    """

    def __init__(self, model_transform_template: ModalContentTransformTemplate, tokenizer=None, max_length: int = 2048,
                 **kwargs):
        self.template = model_transform_template
        self.tokenizer = tokenizer or model_transform_template.tokenizer
        self.template.tokenizer = self.tokenizer
        self.template.check_modal_builder_tokens(self.tokenizer)
        self.max_length = max_length
        self.output_columns = self.template.output_columns

    def __call__(self, query_list: Union[List[dict], List[List[dict]]], history_list=None) -> Dict[str, Any]:
        batch = query_list if query_list and isinstance(query_list[0], (list, tuple)) else [query_list]
        records = [self.template.encode_predict(list(q), i) for i, q in enumerate(batch)]
        out = self.template.batch(records)
        out["input_ids_list"] = [r["input_ids"] for r in records]
        out["raw_query"] = [r["raw_query"] for r in records]
        return out

    @property
    def modal_pad_ids(self) -> List[int]:
        ids = []
        for b in self.template.modal_builders.values():
            if b.need_padding_context:
                b._resolve_ids()
                ids.append(b.context_pad_token_id)
        return ids

    def post_process(self, output_ids, **kwargs) -> List[str]:
        return self.template.post_process(output_ids, **kwargs)

    def decode(self, *args, **kwargs):
        return self.tokenizer.decode(*args, **kwargs)
