"""Token streamers (reference ``generation/streamers.py``): print as text arrives, or iterate from another thread."""
from __future__ import annotations

from queue import Queue
from typing import Optional


class BaseStreamer:
    """Receives tokens as ``generate()`` produces them: ``put(token_ids)`` per step, ``end()`` once (reference
    ``generation/streamers.py``)."""

    def put(self, value):
        raise NotImplementedError

    def end(self):
        raise NotImplementedError


class TextStreamer(BaseStreamer):
    """Decodes incrementally and prints whole words as soon as they are complete."""

    def __init__(self, tokenizer=None, skip_prompt: bool = False, skip_special_tokens: bool = True, **decode_kwargs):
        self.tokenizer, self.skip_prompt = tokenizer, skip_prompt
        self.decode_kwargs = dict(decode_kwargs, skip_special_tokens=skip_special_tokens)
        self.cache, self.print_len, self.next_is_prompt = [], 0, True

    def put(self, value):
        if hasattr(value, "tolist"):
            value = value.tolist()
        if value and isinstance(value[0], (list, tuple)):
            if len(value) > 1:
                raise ValueError("TextStreamer only supports batch size 1")
            value = value[0]
        if self.skip_prompt and self.next_is_prompt:
            self.next_is_prompt = False
            return
        self.next_is_prompt = False
        self.cache.extend(int(v) for v in value)
        text = self.tokenizer.decode(self.cache, **self.decode_kwargs) if self.tokenizer else " ".join(map(str, self.cache))
        if text.endswith("\n"):
            out = text[self.print_len:]
            self.cache, self.print_len = [], 0
        elif text and text[-1] == "�":
            return
        else:
            cut = text.rfind(" ") + 1
            out = text[self.print_len:cut] if cut > self.print_len else ""
            self.print_len += len(out)
        if out:
            self.on_finalized_text(out)

    def end(self):
        if self.cache:
            text = self.tokenizer.decode(self.cache, **self.decode_kwargs) if self.tokenizer else " ".join(map(str, self.cache))
            out = text[self.print_len:]
            self.cache, self.print_len = [], 0
        else:
            out = ""
        self.next_is_prompt = True
        self.on_finalized_text(out, stream_end=True)

    def on_finalized_text(self, text: str, stream_end: bool = False):
        print(text, flush=True, end="" if not stream_end else None)


class TextIteratorStreamer(TextStreamer):
    """Same, but the text pieces are read with ``for piece in streamer`` from another thread."""

    def __init__(self, tokenizer=None, skip_prompt: bool = False, timeout: Optional[float] = None, **kw):
        super().__init__(tokenizer, skip_prompt, **kw)
        self.queue: Queue = Queue()
        self.stop_signal = None
        self.timeout = timeout

    def on_finalized_text(self, text: str, stream_end: bool = False):
        self.queue.put(text, timeout=self.timeout)
        if stream_end:
            self.queue.put(self.stop_signal, timeout=self.timeout)

    def __iter__(self):
        return self

    def __next__(self):
        value = self.queue.get(timeout=self.timeout)
        if value is self.stop_signal:
            raise StopIteration
        return value
