"""Names that the reference's root package exports and that live here under another name."""
from .core.optim import CAME as Came  # noqa: F401
from .tools.logger import logger  # noqa: F401
