"""Weight initialisers (reference ``parallel_core/utils/init_method.py:27-50``)."""
from ...parallel.init_method import init_method_normal, scaled_init_method_normal  # noqa: F401

__all__ = ["init_method_normal", "scaled_init_method_normal"]
