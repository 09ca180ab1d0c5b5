"""Resume helpers under the reference's path (``utils/resume_ckpt_utils.py``)."""
from ..trainer.utils import load_resume_context_from_checkpoint  # noqa: F401
from ..checkpoint.resume import get_resume_checkpoint, record_resume_point, rescale_resume_step  # noqa: F401

__all__ = ["get_resume_checkpoint", "load_resume_context_from_checkpoint", "record_resume_point", "rescale_resume_step"]
