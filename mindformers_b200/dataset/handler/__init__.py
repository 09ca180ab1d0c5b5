"""Data handlers under the reference's ``dataset/handler`` path."""
from ...dataset.handlers import AdgenInstructDataHandler, AlpacaInstructDataHandler, BaseInstructDataHandler, CodeAlpacaInstructDataHandler, LlavaInstructDataHandler, PackingHandler, build_data_handler  # noqa: F401

__all__ = ["AdgenInstructDataHandler", "AlpacaInstructDataHandler", "BaseInstructDataHandler", "CodeAlpacaInstructDataHandler", "LlavaInstructDataHandler", "PackingHandler", "build_data_handler"]
