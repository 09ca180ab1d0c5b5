"""``PagedAttentionMgr`` (reference ``modules/paged_attention_mgr.py``)."""
from ..modules.infer_attention import PagedAttentionMgr  # noqa: F401

__all__ = ["PagedAttentionMgr"]
