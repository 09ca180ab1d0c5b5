"""``KVCacheMgr`` (reference ``modules/kvcache_mgr.py``)."""
from ..modules.infer_attention import KVCacheMgr  # noqa: F401

__all__ = ["KVCacheMgr"]
