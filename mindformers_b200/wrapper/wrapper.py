"""Train-step wrappers (reference ``wrapper/wrapper.py:303,479``)."""
from ..wrapper import MFPipelineWithLossScaleCell, MFTrainOneStepCell  # noqa: F401

__all__ = ["MFPipelineWithLossScaleCell", "MFTrainOneStepCell"]
