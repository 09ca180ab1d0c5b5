"""``load_image``: an image from a path, bytes, a base64 / data-URI string, an http(s) address or a PIL image
(reference ``tools/image_tools.py:27``). Always returns an RGB ``PIL.Image``."""
from __future__ import annotations

import base64
import binascii
import io
import os

from PIL import Image


def load_image(content, timeout: float = 4):
    if isinstance(content, Image.Image):
        return content.convert("RGB")
    if isinstance(content, (bytes, bytearray)):
        return Image.open(io.BytesIO(bytes(content))).convert("RGB")
    if not isinstance(content, str):
        raise TypeError(f"cannot load an image from {type(content).__name__}")
    if content.startswith(("http://", "https://")):
        import urllib.request
        with urllib.request.urlopen(content, timeout=timeout) as resp:      # noqa: S310 (the caller chose the address)
            return Image.open(io.BytesIO(resp.read())).convert("RGB")
    if os.path.isfile(content):
        return Image.open(content).convert("RGB")
    payload = content.split(",", 1)[1] if content.startswith("data:") and "," in content else content
    try:
        return Image.open(io.BytesIO(base64.b64decode(payload, validate=True))).convert("RGB")
    except (binascii.Error, ValueError, OSError) as e:
        raise ValueError("the string is neither an existing file, an http(s) address nor base64 image data") from e
