"""``ModelCommProcessGroups`` (reference ``parallel_core/process_group_config.py:25-123``)."""
from ..parallel.parallel_state import ModelCommProcessGroups  # noqa: F401

__all__ = ["ModelCommProcessGroups"]
