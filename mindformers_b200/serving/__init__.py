"""Online serving: a continuous-batching engine over the paged KV cache and an OpenAI-style HTTP front end."""
from .engine import Request, RequestOutput, SamplingParams, ServingEngine

__all__ = ["Request", "RequestOutput", "SamplingParams", "ServingEngine"]
