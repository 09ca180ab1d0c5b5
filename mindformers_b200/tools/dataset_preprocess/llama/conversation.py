"""Conversation prompt templates (Vicuna-style separators) used when tokenising chat data for Llama models.

Reference: ``tools/dataset_preprocess/llama/conversation.py`` (FastChat-derived ``Conversation`` with
``SeparatorStyle``). Only the styles the Llama preprocessing uses are kept.
"""
from __future__ import annotations

import dataclasses
from enum import Enum, auto
from typing import List, Optional, Tuple


class SeparatorStyle(Enum):
    """How the turns of a conversation template are joined."""

    ADD_COLON_SINGLE = auto()
    ADD_COLON_TWO = auto()
    LLAMA2 = auto()


@dataclasses.dataclass
class Conversation:
    """A prompt template with its history: system text, role names, messages, separators; ``get_prompt()`` renders it
    (reference ``tools/dataset_preprocess/llama/conversation.py``)."""

    name: str
    system: str
    roles: Tuple[str, str]
    messages: List[List[Optional[str]]] = dataclasses.field(default_factory=list)
    sep_style: SeparatorStyle = SeparatorStyle.ADD_COLON_TWO
    sep: str = " "
    sep2: Optional[str] = "</s>"

    def append_message(self, role: str, message: Optional[str]):
        self.messages.append([role, message])

    def copy(self) -> "Conversation":
        return dataclasses.replace(self, messages=[list(m) for m in self.messages])

    def get_prompt(self) -> str:
        if self.sep_style == SeparatorStyle.ADD_COLON_SINGLE:
            out = self.system + self.sep
            for role, msg in self.messages:
                out += f"{role}: {msg}{self.sep}" if msg else f"{role}:"
            return out
        if self.sep_style == SeparatorStyle.ADD_COLON_TWO:
            seps = [self.sep, self.sep2]
            out = self.system + seps[0]
            for i, (role, msg) in enumerate(self.messages):
                out += f"{role}: {msg}{seps[i % 2]}" if msg else f"{role}:"
            return out
        if self.sep_style == SeparatorStyle.LLAMA2:
            out = ""
            for i, (role, msg) in enumerate(self.messages):
                if i % 2 == 0:
                    sys = f"<<SYS>>\n{self.system}\n<</SYS>>\n\n" if i == 0 and self.system else ""
                    out += f"<s>[INST] {sys}{msg} [/INST]"
                elif msg:
                    out += f" {msg} </s>"
            return out
        raise ValueError(self.sep_style)


TEMPLATES = {
    "vicuna_v1.1": Conversation("vicuna_v1.1",
                                "A chat between a curious user and an artificial intelligence assistant. The assistant "
                                "gives helpful, detailed, and polite answers to the user's questions.",
                                ("USER", "ASSISTANT")),
    "llama2": Conversation("llama2", "", ("[INST]", "[/INST]"), sep_style=SeparatorStyle.LLAMA2, sep="", sep2=""),
}


def get_default_conv_template(name: str = "vicuna_v1.1") -> Conversation:
    return TEMPLATES[name].copy()
