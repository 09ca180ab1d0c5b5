"""``pipeline(task, model, tokenizer)`` factory and the text-generation pipelines.

Reference: ``mindformers/pipeline/pipeline.py:59-149`` (factory), ``base_pipeline.py:53-325`` (batching of
list / dataset inputs, preprocess → forward → postprocess) and ``text_generation_pipeline.py:31``.
"""
from __future__ import annotations

from typing import Any, Dict, Iterable, List, Optional, Union

import torch

from ..tools.register.register import MindFormerModuleType, MindFormerRegister

SUPPORTED_TASKS = ("text_generation", "multi_modal_to_text_generation")


class Pipeline:
    """Batches the inputs and runs ``preprocess → _forward → postprocess`` per batch."""

    def __init__(self, model, tokenizer=None, image_processor=None, **kwargs):
        self.model, self.tokenizer, self.image_processor = model, tokenizer, image_processor
        self.default_kwargs = kwargs

    def _sanitize_parameters(self, **kw):
        pre = {k: kw[k] for k in ("add_special_tokens", "max_length_input") if k in kw}
        post = {k: kw[k] for k in ("skip_special_tokens", "return_full_text") if k in kw}
        fwd = {k: v for k, v in kw.items() if k not in pre and k not in post and k != "batch_size"}
        return pre, fwd, post

    def __call__(self, inputs, batch_size: Optional[int] = None, **kwargs):
        merged = dict(self.default_kwargs)
        merged.update(kwargs)
        pre_kw, fwd_kw, post_kw = self._sanitize_parameters(**merged)
        single = isinstance(inputs, (str, dict))
        items = [inputs] if single else list(inputs)
        bs = batch_size or 1
        out: List[Any] = []
        for i in range(0, len(items), bs):
            chunk = items[i:i + bs]
            model_in = self.preprocess(chunk, **pre_kw)
            model_out = self._forward(model_in, **fwd_kw)
            out.extend(self.postprocess(model_out, **post_kw))
        return out[0] if single else out

    def preprocess(self, inputs, **kw):
        raise NotImplementedError

    def _forward(self, model_inputs, **kw):
        raise NotImplementedError

    def postprocess(self, model_outputs, **kw):
        raise NotImplementedError


@MindFormerRegister.register(MindFormerModuleType.PIPELINE, alias="text_generation")
class TextGenerationPipeline(Pipeline):
    """Prompt text (or token ids) in, ``{"text_generation_text": [...]}`` out."""

    def preprocess(self, inputs, add_special_tokens: bool = True, max_length_input: Optional[int] = None, **kw):
        ids = []
        for x in inputs:
            if isinstance(x, str):
                if self.tokenizer is None:
                    raise ValueError("a tokenizer is required for text inputs")
                t = self.tokenizer.encode(x, add_special_tokens=add_special_tokens)
            elif torch.is_tensor(x):
                t = x.tolist()
            else:
                t = list(x)
            ids.append(t[-max_length_input:] if max_length_input else t)
        return {"input_ids": ids}

    @torch.no_grad()
    def _forward(self, model_inputs, **generate_kwargs):
        self.model.eval()
        if self.tokenizer is not None:
            generate_kwargs.setdefault("eos_token_id", getattr(self.tokenizer, "eos_token_id", None))
            generate_kwargs.setdefault("pad_token_id", getattr(self.tokenizer, "pad_token_id", 0) or 0)
        out = self.model.generate(model_inputs["input_ids"], **generate_kwargs)
        return {"output_ids": out, "input_ids": model_inputs["input_ids"]}

    def postprocess(self, model_outputs, skip_special_tokens: bool = True, return_full_text: bool = True, **kw):
        res = []
        for full, prompt in zip(model_outputs["output_ids"], model_outputs["input_ids"]):
            ids = full if return_full_text else full[len(prompt):]
            text = self.tokenizer.decode(ids, skip_special_tokens=skip_special_tokens) if self.tokenizer is not None else ids
            res.append({"text_generation_text": [text]})
        return res


@MindFormerRegister.register(MindFormerModuleType.PIPELINE, alias="multi_modal_to_text_generation")
class MultiModalToTextPipeline(TextGenerationPipeline):
    """Inputs are queries made of parts, ``[{"image": path_or_array}, {"text": "…"}]``.

    With ``processor`` (a ``BaseXModalToTextProcessor``) the parts are tokenised, image placeholders are expanded and
    pixel values with their context positions are passed to ``model.generate`` (reference
    ``pipeline/multi_modal_to_text_generation_pipeline.py``). Without a processor only text parts are accepted and
    the pipeline behaves like text generation.
    """

    def __init__(self, *args, processor=None, **kwargs):
        super().__init__(*args, **kwargs)
        self.processor = processor
        if processor is not None and self.tokenizer is None:
            self.tokenizer = processor.tokenizer

    def preprocess(self, inputs, **kw):
        if self.processor is not None:
            queries = [list(s) if isinstance(s, (list, tuple)) else [s] for s in inputs]
            batch = self.processor(queries)
            out = {"input_ids": batch["input_ids_list"]}
            for k, v in batch.items():
                if k not in ("input_ids", "input_ids_list", "raw_query"):
                    out[k] = v
            return out
        texts = []
        for sample in inputs:
            parts = sample if isinstance(sample, list) else [sample]
            if any(isinstance(p, dict) and "image" in p for p in parts):
                raise ValueError("image parts need processor= (a BaseXModalToTextProcessor) and a multimodal model")
            texts.append("".join(p.get("text", "") if isinstance(p, dict) else str(p) for p in parts))
        return super().preprocess(texts, **kw)

    @torch.no_grad()
    def _forward(self, model_inputs, **generate_kwargs):
        modal = {k: v for k, v in model_inputs.items() if k != "input_ids"}
        if not modal:
            return super()._forward(model_inputs, **generate_kwargs)
        self.model.eval()
        generate_kwargs.setdefault("eos_token_id", getattr(self.tokenizer, "eos_token_id", None))
        out = self.model.generate(model_inputs["input_ids"], **modal, **generate_kwargs)
        return {"output_ids": out, "input_ids": model_inputs["input_ids"]}


class PipelineRegistry:
    """Task table of ``pipeline()`` (reference ``pipeline/pipeline_registry.py:22``): ``supported_tasks`` maps a task name
    to ``{"impl": pipeline class, "ms": model classes, "default": {...}, "type": ...}``, ``task_aliases`` maps other
    spellings to a task name. ``register_pipeline`` adds a task and registers its class for ``pipeline()``."""

    def __init__(self, supported_tasks=None, task_aliases=None):
        self.supported_tasks = dict(supported_tasks or {})
        self.task_aliases = dict(task_aliases or {})

    def get_supported_tasks(self):
        return sorted(set(self.supported_tasks) | set(self.task_aliases))

    def check_task(self, task: str):
        """``(normalised task name, its table entry, None)``; raises ``KeyError`` for an unknown task."""
        task = self.task_aliases.get(task, task)
        if task in self.supported_tasks:
            return task, self.supported_tasks[task], None
        raise KeyError(f"Unknown task {task}, available tasks are {self.get_supported_tasks()}")

    def register_pipeline(self, task: str, pipeline_class, ms_model=None, default=None, task_type=None):
        global SUPPORTED_TASKS
        models = () if ms_model is None else (tuple(ms_model) if isinstance(ms_model, (list, tuple)) else (ms_model,))
        entry = {"impl": pipeline_class, "ms": models}
        if default is not None:
            entry["default"] = default if ("model" in default or "ms" in default) else {"model": default}
        if task_type is not None:
            entry["type"] = task_type
        self.supported_tasks[task] = entry
        pipeline_class.registered_impl = {task: entry}
        bucket = MindFormerRegister.registry.setdefault(MindFormerModuleType.PIPELINE, {})
        bucket[task] = pipeline_class
        if task not in SUPPORTED_TASKS:
            SUPPORTED_TASKS = tuple(SUPPORTED_TASKS) + (task,)

    def to_dict(self):
        return self.supported_tasks


TASK_ALIASES = {"text-generation": "text_generation", "image-to-text": "multi_modal_to_text_generation",
                "image_to_text_generation": "multi_modal_to_text_generation"}


def pipeline(task: Optional[str] = None, model=None, tokenizer=None, image_processor=None, audio_processor=None,
             backend: str = "ms", **kwargs):
    """Build the pipeline for ``task``. ``model`` is a model object, a directory (``from_pretrained``) or a preset name."""
    task = TASK_ALIASES.get(task, task)
    if task not in SUPPORTED_TASKS:
        raise KeyError(f"task {task!r} is not supported; choose from {SUPPORTED_TASKS}")
    if isinstance(model, str):
        from ..models import AutoModel, AutoTokenizer
        path = model
        model = AutoModel.from_pretrained(path)
        if tokenizer is None:
            try:
                tokenizer = AutoTokenizer.from_pretrained(path)
            except Exception:
                tokenizer = None
    if model is None:
        raise ValueError("pipeline() needs a model")
    cls = MindFormerRegister.get_cls(MindFormerModuleType.PIPELINE, task)
    return cls(model=model, tokenizer=tokenizer, image_processor=image_processor, **kwargs)


PIPELINE_REGISTRY = PipelineRegistry(
    {"text_generation": {"impl": TextGenerationPipeline, "ms": (), "type": "text"},
     "multi_modal_to_text_generation": {"impl": MultiModalToTextPipeline, "ms": (), "type": "multimodal"}}, TASK_ALIASES)


# ``mindformers_b200.pipeline`` names both this package and the factory function above. Calling the package calls the
# function, so ``from mindformers_b200 import pipeline; pipeline("text_generation", ...)`` works whichever of the two
# the import machinery hands out, and ``import mindformers_b200.pipeline as pl; pl.pipeline`` keeps meaning the module.
import sys as _sys
import types as _types


class _CallablePackage(_types.ModuleType):
    def __call__(self, *args, **kwargs):
        return pipeline(*args, **kwargs)


_sys.modules[__name__].__class__ = _CallablePackage

from .._submodules import keep_functions as _keep_functions  # noqa: E402

_keep_functions(__name__, ('pipeline',))
