"""``MFModelConfig`` (reference ``parallel_core/mf_model_config.py``): there a separate dataclass for the framework's own
knobs (compute / norm / rotary / softmax dtypes, ``use_flash_attention``, ``input_layout``, ``use_ring_attention``,
``mla_qkv_concat``, ...) that ``TransformerConfig`` inherits next to ``ModelParallelConfig``. Here those fields are
declared directly on ``TransformerConfig``; the name is kept for code that annotates or checks against it."""
from ..parallel.transformer_config import TransformerConfig  # noqa: F401

MFModelConfig = TransformerConfig

__all__ = ["MFModelConfig"]
