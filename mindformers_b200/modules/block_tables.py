"""``BlockTables`` (reference ``modules/block_tables.py:65-121``)."""
from ..inference.block_manager import BlockTables  # noqa: F401

__all__ = ["BlockTables"]
