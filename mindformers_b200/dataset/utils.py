"""Dataset configuration checks (reference ``dataset/utils.py``)."""
from ..dataset.base_dataset import check_dataset_config, check_dataset_iterable, is_generator_function  # noqa: F401

__all__ = ["check_dataset_config", "check_dataset_iterable", "is_generator_function"]
