"""``build_wrapper`` (reference ``wrapper/build_wrapper.py``)."""
from ..tools.register import MindFormerModuleType, MindFormerRegister
from . import MFPipelineWithLossScaleCell, MFTrainOneStepCell  # noqa: F401  (registers the classes)


def build_wrapper(config=None, default_args=None, class_name=None, **kwargs):
    """A train-step wrapper from ``{"type": name, ...}`` or from ``class_name`` and keyword arguments."""
    if config is None and class_name is None:
        return None
    if config is not None:
        return MindFormerRegister.get_instance_from_cfg(dict(config), MindFormerModuleType.WRAPPER, default_args=default_args)
    return MindFormerRegister.get_instance(MindFormerModuleType.WRAPPER, class_name, **kwargs)
