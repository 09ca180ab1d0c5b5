"""``@deprecated`` for functions and classes (reference ``mindformers/utils/decorators.py``)."""
from __future__ import annotations

import functools
import inspect
import warnings
from typing import Optional


def deprecated(reason: Optional[str] = None, version: Optional[str] = None, removal: Optional[str] = None):
    """Warn once per call site with ``DeprecationWarning``. Usable bare (``@deprecated``) or with arguments."""

    def build(obj, why):
        kind = "class" if inspect.isclass(obj) else "function"
        msg = f"{kind} {obj.__qualname__} is deprecated"
        if version:
            msg += f" since {version}"
        if removal:
            msg += f" and will be removed in {removal}"
        if why:
            msg += f": {why}"
        if inspect.isclass(obj):
            init = obj.__init__

            @functools.wraps(init)
            def new_init(self, *a, **k):
                warnings.warn(msg, DeprecationWarning, stacklevel=2)
                init(self, *a, **k)

            obj.__init__ = new_init
            return obj

        @functools.wraps(obj)
        def wrapper(*a, **k):
            warnings.warn(msg, DeprecationWarning, stacklevel=2)
            return obj(*a, **k)

        return wrapper

    if callable(reason):            # bare @deprecated
        return build(reason, None)
    return lambda obj: build(obj, reason)
