"""Data handlers under the reference's ``dataset/handler`` path."""
from ...dataset.handlers import (AdgenInstructDataHandler, AlpacaInstructDataHandler, BaseInstructDataHandler,  # noqa: F401
                                 CodeAlpacaInstructDataHandler, LlavaInstructDataHandler, PackingConfig, PackingHandler,
                                 build_data_handler, pack_examples, truncate_examples)

__all__ = ["AdgenInstructDataHandler", "AlpacaInstructDataHandler", "BaseInstructDataHandler", "CodeAlpacaInstructDataHandler",
           "LlavaInstructDataHandler", "PackingConfig", "PackingHandler", "build_data_handler", "pack_examples", "truncate_examples"]
