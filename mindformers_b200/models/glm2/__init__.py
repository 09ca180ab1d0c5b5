"""The ChatGLM2 / 3 / GLM-4 family under its reference import path (``mindformers/models/glm2``)."""
from ...models.families import ChatGLM2Config, ChatGLM2ForConditionalGeneration, ChatGLM2Model, ChatGLM2WithPtuning2  # noqa: F401
from ...models.tokenizers import ChatGLM2Tokenizer, ChatGLM3Tokenizer, ChatGLM4Tokenizer  # noqa: F401
from ...models.processing_utils import GLMProcessor  # noqa: F401

__all__ = ["ChatGLM2Config", "ChatGLM2ForConditionalGeneration", "ChatGLM2Model", "ChatGLM2Tokenizer", "ChatGLM2WithPtuning2",
           "ChatGLM3Tokenizer", "ChatGLM4Tokenizer", "GLMProcessor"]
