"""``BaseConfig``: older name of the configuration base class (reference ``models/base_config.py``)."""
from ..models.configuration_utils import PretrainedConfig  # noqa: F401
BaseConfig = PretrainedConfig

__all__ = ["PretrainedConfig"]
