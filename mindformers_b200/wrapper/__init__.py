"""Train-step wrappers under the reference's names.

``MFTrainOneStepCell`` (``mindformers/wrapper/wrapper.py:303``) = forward + backward + gradient clipping + loss scaling
+ optimizer step for a model that is not pipeline-staged; ``MFPipelineWithLossScaleCell`` (``:780``) = the same over a
pipeline schedule. Here they are ``TrainOneStep`` and ``PipelineTrainStep``; the aliases let configs and user code
that name the reference's classes resolve.
"""
from ..parallel.distributed.train_step import TrainOneStep
from ..parallel.pipeline import PipelineTrainStep
from ..tools.register import MindFormerModuleType, MindFormerRegister
from .micro_batch_interleave import MicroBatchInterleaved

MFTrainOneStepCell = TrainOneStep
MFPipelineWithLossScaleCell = PipelineTrainStep

for _name, _cls in (("MFTrainOneStepCell", TrainOneStep), ("MFPipelineWithLossScaleCell", PipelineTrainStep)):
    if not MindFormerRegister.is_exist(MindFormerModuleType.WRAPPER, _name):
        MindFormerRegister.register_cls(_cls, MindFormerModuleType.WRAPPER, alias=_name)

__all__ = ["MFTrainOneStepCell", "MFPipelineWithLossScaleCell", "TrainOneStep", "PipelineTrainStep", "MicroBatchInterleaved"]
