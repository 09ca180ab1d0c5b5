"""``build_pipeline`` (reference ``pipeline/build_pipeline.py``)."""
from ..tools.register import MindFormerModuleType, MindFormerRegister
from . import MultiModalToTextPipeline, TextGenerationPipeline  # noqa: F401  (registers the classes)


def build_pipeline(config=None, default_args=None, class_name=None, **kwargs):
    """A pipeline from ``{"type": name, ...}`` or from ``class_name`` and keyword arguments."""
    if config is None and class_name is None:
        return None
    if config is not None:
        return MindFormerRegister.get_instance_from_cfg(dict(config), MindFormerModuleType.PIPELINE, default_args=default_args)
    return MindFormerRegister.get_instance(MindFormerModuleType.PIPELINE, class_name, **kwargs)
