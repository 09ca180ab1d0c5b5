"""``ModuleSpec`` / ``build_module`` (reference ``parallel_core/utils/spec_utils.py``)."""
from ...parallel.spec_utils import ModuleSpec, build_module  # noqa: F401

__all__ = ["ModuleSpec", "build_module"]
