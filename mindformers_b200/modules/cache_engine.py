"""``BlockMemPool`` / ``CacheEngine`` (reference ``modules/cache_engine.py:20-90``)."""
from ..inference.block_manager import BlockMemPool, CacheEngine  # noqa: F401

__all__ = ["BlockMemPool", "CacheEngine"]
