"""Process groups (reference ``parallel_core/inference/parallel_state.py``)."""
from ...parallel.parallel_state import *  # noqa: F401,F403
