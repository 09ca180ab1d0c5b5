from .config import ActionDict, DictConfig, MindFormerConfig, parse_value
from .register import MindFormerModuleType, MindFormerRegister, is_legacy_mode, set_use_legacy
from .template import ConfigTemplate

__all__ = ["ActionDict", "DictConfig", "MindFormerConfig", "parse_value", "MindFormerModuleType", "MindFormerRegister",
           "ConfigTemplate", "is_legacy_mode", "set_use_legacy"]
