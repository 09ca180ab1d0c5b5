"""Concrete tokenizers of the supported model families.

* ``LlamaTokenizer`` — sentencepiece ``tokenizer.model`` (reference ``models/llama/llama_tokenizer.py``).
* ``LlamaTokenizerFast`` — a ``tokenizer.json`` run by the ``tokenizers`` library
  (reference ``models/llama/llama_tokenizer_fast.py``); also what DeepSeek-V3 / Qwen3 HF directories ship.
* ``Llama3Tokenizer`` — tiktoken rank file + 256 reserved specials (reference ``research/llama3_1/llama3_1_tokenizer.py``).
* ``Qwen2Tokenizer`` — ``vocab.json`` + ``merges.txt`` byte-level BPE with ``<|im_start|>`` chat markers
  (reference ``research/qwen2_5/qwen2_5_tokenizer.py``).
* ``ChatGLM3Tokenizer`` / ``ChatGLM4Tokenizer`` — sentencepiece resp. tiktoken vocabulary with role tokens, left
  padding and ``build_chat_input`` (reference ``models/glm2/glm3_tokenizer.py``, ``glm4_tokenizer.py``).
* ``TelechatTokenizer`` — sentencepiece with ``<_user>`` / ``<_bot>`` markers (reference ``research/telechat2``).

All byte-level BPE tokenizers run on ``BytePairEncoder`` of ``tokenization_utils``.
"""
from __future__ import annotations

import json
import os
import shutil
from typing import Dict, List, Optional, Union

from ..tools.register import MindFormerModuleType, MindFormerRegister
from .tokenization_utils import (AddedToken, BytePairEncoder, PreTrainedTokenizer, bytes_to_unicode, load_gpt2_ranks,
                                 load_tiktoken_ranks, save_tiktoken_ranks)

LLAMA3_PATTERN = (r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n]*|"
                  r"\s*[\r\n]+|\s+(?!\S)|\s+")
QWEN2_PATTERN = (r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*|"
                 r"\s*[\r\n]+|\s+(?!\S)|\s+")

LLAMA3_CHAT_TEMPLATE = (
    "{% for message in messages %}"
    "{% set content = '<|start_header_id|>' + message['role'] + '<|end_header_id|>\n\n' + message['content'] | trim + '<|eot_id|>' %}"
    "{% if loop.index0 == 0 %}{% set content = bos_token + content %}{% endif %}"
    "{{ content }}"
    "{% endfor %}"
    "{% if add_generation_prompt %}{{ '<|start_header_id|>assistant<|end_header_id|>\n\n' }}{% endif %}")
CHATML_TEMPLATE = (
    "{% for message in messages %}"
    "{% if loop.first and message['role'] != 'system' %}{{ '<|im_start|>system\nYou are a helpful assistant.<|im_end|>\n' }}{% endif %}"
    "{{ '<|im_start|>' + message['role'] + '\n' + message['content'] + '<|im_end|>' + '\n' }}"
    "{% endfor %}"
    "{% if add_generation_prompt %}{{ '<|im_start|>assistant\n' }}{% endif %}")
LLAMA2_CHAT_TEMPLATE = (
    "{% for message in messages %}"
    "{% if message['role'] == 'user' %}{{ bos_token + '[INST] ' + message['content'] | trim + ' [/INST]' }}"
    "{% elif message['role'] == 'system' %}{{ '<<SYS>>\n' + message['content'] | trim + '\n<</SYS>>\n\n' }}"
    "{% elif message['role'] == 'assistant' %}{{ ' ' + message['content'] | trim + ' ' + eos_token }}{% endif %}"
    "{% endfor %}")


class _SentencePieceMixin:
    """Shared plumbing of the sentencepiece-backed tokenizers."""

    def _load_sp(self, vocab_file: str):
        import sentencepiece as spm
        if not vocab_file or not os.path.isfile(vocab_file):
            raise FileNotFoundError(f"sentencepiece model {vocab_file!r} not found")
        self.vocab_file = vocab_file
        self.sp_model = spm.SentencePieceProcessor()
        self.sp_model.Load(vocab_file)

    @property
    def vocab_size(self) -> int:
        return self.sp_model.GetPieceSize()

    def _convert_token_to_id(self, token):
        return self.sp_model.PieceToId(token)

    def _convert_id_to_token(self, index: int):
        return self.sp_model.IdToPiece(int(index)) if 0 <= index < self.vocab_size else ""

    def save_vocabulary(self, save_directory: str, filename_prefix: Optional[str] = None):
        name = (f"{filename_prefix}-" if filename_prefix else "") + self.vocab_files_names["vocab_file"]
        dst = os.path.join(save_directory, name)
        if os.path.abspath(dst) != os.path.abspath(self.vocab_file):
            if os.path.isfile(self.vocab_file):
                shutil.copyfile(self.vocab_file, dst)
            else:
                with open(dst, "wb") as f:
                    f.write(self.sp_model.serialized_model_proto())
        return (dst,)

    def __getstate__(self):
        state = self.__dict__.copy()
        state["sp_model"] = None
        return state

    def __setstate__(self, state):
        self.__dict__.update(state)
        self._load_sp(self.vocab_file)


@MindFormerRegister.register(MindFormerModuleType.TOKENIZER)
class LlamaTokenizer(_SentencePieceMixin, PreTrainedTokenizer):
    """SentencePiece tokenizer of Llama / Llama 2 (reference ``models/llama/llama_tokenizer.py``): ``tokenizer.model``,
    optional BOS / EOS insertion, the Llama 2 chat template."""

    vocab_files_names = {"vocab_file": "tokenizer.model"}
    default_chat_template = LLAMA2_CHAT_TEMPLATE

    def __init__(self, vocab_file: str, unk_token="<unk>", bos_token="<s>", eos_token="</s>", pad_token="<unk>",
                 add_bos_token: bool = True, add_eos_token: bool = False, legacy: bool = True, **kwargs):
        self._load_sp(vocab_file)
        self.legacy = legacy
        super().__init__(vocab_file=vocab_file, unk_token=unk_token, bos_token=bos_token, eos_token=eos_token,
                         pad_token=pad_token, add_bos_token=add_bos_token, add_eos_token=add_eos_token, **kwargs)

    def _tokenize(self, text: str, **kwargs) -> List[str]:
        return self.sp_model.EncodeAsPieces(text)

    def convert_tokens_to_string(self, tokens: List[str]) -> str:
        return self.sp_model.DecodePieces(list(tokens))


@MindFormerRegister.register(MindFormerModuleType.TOKENIZER)
class TelechatTokenizer(LlamaTokenizer):
    """SentencePiece tokenizer of TeleChat with its ``<_user>`` / ``<_bot>`` / ``<_system>`` role tokens (reference
    ``research/telechat2/telechat_tokenizer.py``)."""

    def __init__(self, vocab_file: str, unk_token="<unk>", bos_token="<_start>", eos_token="<_end>",
                 pad_token="<_pad>", add_bos_token: bool = False, add_eos_token: bool = False, **kwargs):
        kwargs.setdefault("additional_special_tokens", ["<_user>", "<_bot>", "<_system>"])
        super().__init__(vocab_file, unk_token=unk_token, bos_token=bos_token, eos_token=eos_token,
                         pad_token=pad_token, add_bos_token=add_bos_token, add_eos_token=add_eos_token, **kwargs)

    def build_chat_input(self, query: str, history: Optional[List[Dict[str, str]]] = None, system: str = ""):
        text = (f"<_system>{system}" if system else "")
        for turn in history or []:
            text += ("<_user>" if turn["role"] == "user" else "<_bot>") + turn["content"]
            if turn["role"] != "user":
                text += str(self.eos_token)
        text += f"<_user>{query}<_bot>"
        return self(text, add_special_tokens=False)


class PreTrainedTokenizerFast(PreTrainedTokenizer):
    """Base of the tokenizers that run on the ``tokenizers`` library (reference ``models/tokenization_utils_fast.py``):
    built from a ``tokenizer.json`` file, from a ``tokenizers.Tokenizer`` object, or from a slow tokenizer through
    ``convert_slow_tokenizer`` (``slow_tokenizer=``)."""
    vocab_files_names = {"tokenizer_file": "tokenizer.json"}
    slow_tokenizer_class = None

    def __init__(self, tokenizer_file: Optional[str] = None, bos_token=None, eos_token=None, unk_token=None, pad_token=None,
                 add_bos_token: bool = False, add_eos_token: bool = False, tokenizer_object=None, slow_tokenizer=None,
                 **kwargs):
        from tokenizers import Tokenizer
        self.tokenizer_file = tokenizer_file
        if tokenizer_object is not None:
            self.backend = tokenizer_object
        elif slow_tokenizer is not None:
            self.backend = convert_slow_tokenizer(slow_tokenizer)
            bos_token = bos_token or slow_tokenizer.bos_token
            eos_token = eos_token or slow_tokenizer.eos_token
            unk_token = unk_token or slow_tokenizer.unk_token
            pad_token = pad_token or slow_tokenizer.pad_token
        elif tokenizer_file is not None:
            self.backend = Tokenizer.from_file(tokenizer_file)
        else:
            raise ValueError("one of tokenizer_file, tokenizer_object or slow_tokenizer is required")
        super().__init__(tokenizer_file=tokenizer_file, bos_token=bos_token, eos_token=eos_token, unk_token=unk_token,
                         pad_token=pad_token, add_bos_token=add_bos_token, add_eos_token=add_eos_token, **kwargs)

    @property
    def vocab_size(self) -> int:
        return self.backend.get_vocab_size(with_added_tokens=True)

    def get_vocab(self):
        return self.backend.get_vocab(with_added_tokens=True)

    def _tokenize(self, text: str, **kwargs):
        return self.backend.encode(text, add_special_tokens=False).tokens

    def tokenize(self, text: str, **kwargs):
        return self._tokenize(text)          # the backend splits its own added tokens

    def _to_ids(self, text, **kwargs):
        if isinstance(text, str):
            return self.backend.encode(text, add_special_tokens=False).ids
        return super()._to_ids(text, **kwargs)

    def _convert_token_to_id(self, token):
        return self.backend.token_to_id(token)

    def _convert_id_to_token(self, index: int):
        return self.backend.id_to_token(int(index))

    def convert_tokens_to_string(self, tokens):
        return self.backend.decode([self.backend.token_to_id(t) for t in tokens], skip_special_tokens=False)

    def _decode(self, token_ids, skip_special_tokens: bool = False, **kwargs):
        return self.backend.decode([int(i) for i in token_ids], skip_special_tokens=skip_special_tokens)

    def add_tokens(self, new_tokens, special_tokens: bool = False) -> int:
        from tokenizers import AddedToken as FastAdded
        if isinstance(new_tokens, (str, AddedToken)):
            new_tokens = [new_tokens]
        toks = [FastAdded(str(t), special=special_tokens, normalized=False) for t in new_tokens if str(t)]
        if not toks:
            return 0
        return self.backend.add_special_tokens(toks) if special_tokens else self.backend.add_tokens(toks)

    def __len__(self):
        return self.vocab_size

    def save_vocabulary(self, save_directory: str, filename_prefix: Optional[str] = None):
        name = (f"{filename_prefix}-" if filename_prefix else "") + "tokenizer.json"
        dst = os.path.join(save_directory, name)
        self.backend.save(dst)
        return (dst,)


@MindFormerRegister.register(MindFormerModuleType.TOKENIZER)
class LlamaTokenizerFast(PreTrainedTokenizerFast):
    """``tokenizer.json`` of the Llama family run by the ``tokenizers`` library."""


def merges_from_ranks(ranks: Dict[bytes, int]):
    """The merge list that a rank table implies: a token of two or more bytes was formed by joining the two parts that
    byte-pair encoding yields for it when only lower-ranked merges are allowed. Returned in rank order."""
    merges = []
    for token, rank in sorted(ranks.items(), key=lambda kv: kv[1]):
        if len(token) < 2:
            continue
        parts = [bytes([b]) for b in token]
        while len(parts) > 2:
            best, best_rank = None, None
            for i in range(len(parts) - 1):
                r = ranks.get(parts[i] + parts[i + 1])
                if r is not None and r < rank and (best_rank is None or r < best_rank):
                    best, best_rank = i, r
            if best is None:
                break
            parts[best:best + 2] = [parts[best] + parts[best + 1]]
        if len(parts) == 2:
            merges.append((parts[0], parts[1]))
    return merges


def convert_slow_tokenizer(slow):
    """A ``tokenizers.Tokenizer`` that encodes like ``slow`` (reference ``models/convert_slow_tokenizer.py``).

    Byte-level BPE tokenizers (rank table + split pattern: Llama-3, Qwen2, GLM-4 styles) become a ``BPE`` model over
    the printable-character alphabet with a regex ``Split`` + ``ByteLevel`` pre-tokenizer and their special tokens
    added; sentencepiece-backed tokenizers are converted from their ``.model`` file by the library's own importer."""
    from tokenizers import AddedToken as FastAdded, Regex, Tokenizer, decoders, models, pre_tokenizers
    if isinstance(slow, _TiktokenStyle):
        table = bytes_to_unicode()
        uni = lambda tok: "".join(table[b] for b in tok)
        vocab = {uni(tok): idx for tok, idx in slow.mergeable_ranks.items()}
        merges = [(uni(a), uni(b)) for a, b in merges_from_ranks(slow.mergeable_ranks)]
        backend = Tokenizer(models.BPE(vocab=vocab, merges=merges, fuse_unk=False, byte_fallback=False,
                                       ignore_merges=False))
        backend.pre_tokenizer = pre_tokenizers.Sequence([
            pre_tokenizers.Split(Regex(slow.pattern), behavior="isolated", invert=False),
            pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)])
        backend.decoder = decoders.ByteLevel()
        specials = sorted(slow.special_tokens.items(), key=lambda kv: kv[1])
        next_id = len(vocab)
        for tok, idx in specials:
            if idx != next_id:
                raise ValueError(f"special token {tok!r} has id {idx}, but the fast vocabulary would give it {next_id}: "
                                 "special tokens must follow the ordinary ones without gaps")
            next_id += 1
        backend.add_special_tokens([FastAdded(t, special=True, normalized=False) for t, _ in specials])
        return backend
    sp_file = getattr(slow, "vocab_file", None)
    if sp_file and str(sp_file).endswith(".model"):
        from tokenizers.implementations import SentencePieceUnigramTokenizer
        return SentencePieceUnigramTokenizer.from_spm(sp_file)._tokenizer
    raise TypeError(f"no conversion for {type(slow).__name__}")


class _TiktokenStyle(PreTrainedTokenizer):
    """Byte-level BPE over a rank table; tokens are ``bytes`` (ordinary) or ``str`` (special)."""
    pattern = LLAMA3_PATTERN

    def _setup_bpe(self, ranks: Dict[bytes, int], special_tokens: Dict[str, int]):
        self.mergeable_ranks = ranks
        self.special_tokens = dict(special_tokens)
        self._id_to_special = {v: k for k, v in special_tokens.items()}
        self.bpe = BytePairEncoder(ranks, self.pattern)

    @property
    def vocab_size(self) -> int:
        return len(self.mergeable_ranks) + len(self.special_tokens)

    def get_vocab(self):
        vocab: Dict[Union[bytes, str], int] = dict(self.mergeable_ranks)
        vocab.update(self.special_tokens)
        vocab.update(self.added_tokens_encoder)
        return vocab

    def _splitter(self):
        if self._split_re is None:
            import regex as re
            toks = sorted(set(self.special_tokens) | set(self.added_tokens_encoder), key=len, reverse=True)
            self._split_re = re.compile("(" + "|".join(re.escape(t) for t in toks) + ")") if toks else None
        return self._split_re

    def _tokenize(self, text: str, **kwargs) -> List[bytes]:
        return [self.bpe.decoder[i] for i in self.bpe.encode_ordinary(text)]

    def _convert_token_to_id(self, token):
        if isinstance(token, str):
            if token in self.special_tokens:
                return self.special_tokens[token]
            token = token.encode("utf-8")
        return self.mergeable_ranks.get(token)

    def _convert_id_to_token(self, index: int):
        index = int(index)
        if index in self._id_to_special:
            return self._id_to_special[index]
        return self.bpe.decoder.get(index, b"")

    def convert_tokens_to_string(self, tokens) -> str:
        out, buf = [], b""
        for t in tokens:
            if isinstance(t, bytes):
                buf += t
            else:
                if buf:
                    out.append(buf.decode("utf-8", errors="replace"))
                    buf = b""
                out.append(t)
        if buf:
            out.append(buf.decode("utf-8", errors="replace"))
        return "".join(out)

    @property
    def all_special_ids(self) -> List[int]:
        return sorted(set(self.special_tokens.values()) | set(super().all_special_ids))

    def save_vocabulary(self, save_directory: str, filename_prefix: Optional[str] = None):
        name = (f"{filename_prefix}-" if filename_prefix else "") + self.vocab_files_names["vocab_file"]
        dst = os.path.join(save_directory, name)
        save_tiktoken_ranks(self.mergeable_ranks, dst)
        return (dst,)


def _ranks_from_tokenizer_json(path: str) -> Dict[bytes, int]:
    """The ``model.vocab`` of an HF ``tokenizer.json`` (printable-character form) as a rank table."""
    with open(path, "r", encoding="utf-8") as f:
        vocab = json.load(f)["model"]["vocab"]
    inv = {c: b for b, c in bytes_to_unicode().items()}
    return {bytes(inv[c] for c in tok): idx for tok, idx in vocab.items() if all(c in inv for c in tok)}


@MindFormerRegister.register(MindFormerModuleType.TOKENIZER)
class Llama3Tokenizer(_TiktokenStyle):
    """Llama 3 / 3.1 tokenizer (reference ``research/llama3_1/llama3_1_tokenizer.py``): tiktoken-style byte-pair
    ranks, the 256 reserved special tokens, the header / end-of-turn chat template."""

    vocab_files_names = {"vocab_file": "tokenizer.model"}
    default_chat_template = LLAMA3_CHAT_TEMPLATE

    def __init__(self, vocab_file: str, bos_token="<|begin_of_text|>", eos_token="<|end_of_text|>",
                 pad_token="<|reserved_special_token_0|>", add_bos_token: bool = False, add_eos_token: bool = False,
                 num_reserved_special_tokens: int = 256, **kwargs):
        ranks = _ranks_from_tokenizer_json(vocab_file) if vocab_file.endswith(".json") else load_tiktoken_ranks(vocab_file)
        names = ["<|begin_of_text|>", "<|end_of_text|>", "<|reserved_special_token_0|>", "<|reserved_special_token_1|>",
                 "<|reserved_special_token_2|>", "<|reserved_special_token_3|>", "<|start_header_id|>",
                 "<|end_header_id|>", "<|reserved_special_token_4|>", "<|eot_id|>"]
        names += [f"<|reserved_special_token_{i}|>" for i in range(5, num_reserved_special_tokens - 5)]
        self._setup_bpe(ranks, {t: len(ranks) + i for i, t in enumerate(names)})
        self.vocab_file = vocab_file
        super().__init__(vocab_file=vocab_file, bos_token=bos_token, eos_token=eos_token, pad_token=pad_token,
                         add_bos_token=add_bos_token, add_eos_token=add_eos_token,
                         num_reserved_special_tokens=num_reserved_special_tokens, **kwargs)


@MindFormerRegister.register(MindFormerModuleType.TOKENIZER)
class Qwen2Tokenizer(_TiktokenStyle):
    """Byte-level BPE tokenizer of Qwen2 / Qwen2.5 / Qwen3 (reference ``research/qwen2_5/qwen2_5_tokenizer.py``):
    ``vocab.json`` + ``merges.txt``, ``<|im_start|>`` / ``<|im_end|>`` ChatML template."""

    vocab_files_names = {"vocab_file": "vocab.json", "merges_file": "merges.txt"}
    pattern = QWEN2_PATTERN
    default_chat_template = CHATML_TEMPLATE

    def __init__(self, vocab_file: str, merges_file: Optional[str] = None, unk_token="<|endoftext|>", bos_token=None,
                 eos_token="<|endoftext|>", pad_token="<|endoftext|>", add_bos_token: bool = False,
                 add_eos_token: bool = False, **kwargs):
        ranks = load_gpt2_ranks(vocab_file, merges_file)
        with open(vocab_file, "r", encoding="utf-8") as f:
            raw = json.load(f)
        base = max(ranks.values()) + 1 if ranks else 0
        special = {}
        for i, t in enumerate(["<|endoftext|>", "<|im_start|>", "<|im_end|>"]):
            special[t] = raw.get(t, base + i)     # 151643..151645 with the released vocabulary
        self._setup_bpe(ranks, special)
        self.vocab_file, self.merges_file = vocab_file, merges_file
        self._raw_vocab = raw
        super().__init__(vocab_file=vocab_file, merges_file=merges_file, unk_token=unk_token, bos_token=bos_token,
                         eos_token=eos_token, pad_token=pad_token, add_bos_token=add_bos_token,
                         add_eos_token=add_eos_token, **kwargs)
        self.end_of_text_id = self.special_tokens["<|endoftext|>"]
        self.im_start_id, self.im_end_id = self.special_tokens["<|im_start|>"], self.special_tokens["<|im_end|>"]

    def prepare_for_tokenization(self, text, **kwargs):
        import unicodedata
        return unicodedata.normalize("NFC", text), kwargs

    def save_vocabulary(self, save_directory: str, filename_prefix: Optional[str] = None):
        prefix = f"{filename_prefix}-" if filename_prefix else ""
        table = bytes_to_unicode()
        vocab = {"".join(table[b] for b in tok): idx for tok, idx in self.mergeable_ranks.items()}
        vpath = os.path.join(save_directory, prefix + "vocab.json")
        with open(vpath, "w", encoding="utf-8") as f:
            json.dump(vocab, f, ensure_ascii=False)
        mpath = os.path.join(save_directory, prefix + "merges.txt")
        if self.merges_file and os.path.exists(self.merges_file):
            if os.path.abspath(self.merges_file) != os.path.abspath(mpath):
                shutil.copyfile(self.merges_file, mpath)
        else:
            with open(mpath, "w", encoding="utf-8") as f:
                f.write("#version: 0.2\n")
        return (vpath, mpath)


class _GLMChatMixin:
    """Role tokens, ``[gMASK] sop`` prefix, left padding with position ids (GLM-3 / GLM-4)."""
    padding_side = "left"
    model_input_names = ["input_ids", "attention_mask", "position_ids"]

    def get_command(self, token: str) -> int:
        idx = self.convert_tokens_to_ids(token)
        if idx is None:
            raise KeyError(f"{token} is not a special token of {type(self).__name__}")
        return idx

    def get_prefix_tokens(self) -> List[int]:
        return [self.get_command("[gMASK]"), self.get_command("sop")]

    def build_inputs_with_special_tokens(self, token_ids_0, token_ids_1=None):
        out = self.get_prefix_tokens() + list(token_ids_0)
        if token_ids_1 is not None:
            out = out + list(token_ids_1) + [self.get_command("<eos>") if self.convert_tokens_to_ids("<eos>") is not None
                                             else self.eos_token_id]
        return out

    def build_single_message(self, role: str, metadata: str, message: str) -> List[int]:
        if role not in ("system", "user", "assistant", "observation"):
            raise ValueError(f"unknown role {role!r}")
        head = [self.get_command(f"<|{role}|>")] + self._to_ids(f"{metadata}\n")
        return head + self._to_ids(message)

    def build_chat_input(self, query: str, history: Optional[List[Dict[str, str]]] = None, role: str = "user",
                         return_tensors: Optional[str] = "pt"):
        ids: List[int] = []
        for item in history or []:
            content = item["content"]
            if item["role"] == "system" and "tools" in item:
                content = content + "\n" + json.dumps(item["tools"], indent=4, ensure_ascii=False)
            ids.extend(self.build_single_message(item["role"], item.get("metadata", ""), content))
        ids.extend(self.build_single_message(role, "", query))
        ids.append(self.get_command("<|assistant|>"))
        ids = self.get_prefix_tokens() + ids
        row = {"input_ids": ids, "attention_mask": [1] * len(ids), "position_ids": list(range(len(ids)))}
        return self._tensors(type(self).pad(self, [row], padding=False), return_tensors)

    def _pad_one(self, enc, width, side):
        n = len(enc["input_ids"])
        enc.setdefault("attention_mask", [1] * n)
        enc.setdefault("position_ids", list(range(n)))
        return super()._pad_one(enc, width, "left")


@MindFormerRegister.register(MindFormerModuleType.TOKENIZER)
class ChatGLM3Tokenizer(_GLMChatMixin, _SentencePieceMixin, PreTrainedTokenizer):
    """SentencePiece tokenizer of ChatGLM3 (reference ``models/glm2/glm3_tokenizer.py``): role tokens appended after
    the SentencePiece vocabulary, ``[gMASK] sop`` prefix, ``build_chat_input``."""

    vocab_files_names = {"vocab_file": "tokenizer.model"}
    ROLE_TOKENS = ["[MASK]", "[gMASK]", "[sMASK]", "sop", "eop", "<|system|>", "<|user|>", "<|assistant|>",
                   "<|observation|>"]

    def __init__(self, vocab_file: str, bos_token="<s>", eos_token="</s>", unk_token="<unk>", pad_token="<unk>",
                 **kwargs):
        self._load_sp(vocab_file)
        kwargs.setdefault("additional_special_tokens", list(self.ROLE_TOKENS))
        kwargs.pop("add_bos_token", None)
        kwargs.pop("add_eos_token", None)
        super().__init__(vocab_file=vocab_file, bos_token=bos_token, eos_token=eos_token, unk_token=unk_token,
                         pad_token=pad_token, **kwargs)

    def _tokenize(self, text: str, **kwargs):
        return self.sp_model.EncodeAsPieces(text)

    def convert_tokens_to_string(self, tokens):
        return self.sp_model.DecodePieces(list(tokens))


@MindFormerRegister.register(MindFormerModuleType.TOKENIZER)
class ChatGLM2Tokenizer(ChatGLM3Tokenizer):
    """SentencePiece tokenizer of ChatGLM2 (reference ``models/glm2/glm2_tokenizer.py``): the five command tokens
    ``[MASK] [gMASK] [sMASK] sop eop`` follow the SentencePiece vocabulary (no role tokens), inputs start with
    ``[gMASK] sop``, and a chat is written as numbered rounds by ``build_prompt``."""

    ROLE_TOKENS = ["[MASK]", "[gMASK]", "[sMASK]", "sop", "eop"]

    def build_prompt(self, query: str, history=None) -> str:
        prompt = ""
        history = history or []
        for i, (old_query, response) in enumerate(history):
            prompt += "[Round {}]\n\n问：{}\n\n答：{}\n\n".format(i + 1, old_query, response)
        return prompt + "[Round {}]\n\n问：{}\n\n答：".format(len(history) + 1, query)

    def build_chat_input(self, query: str, history=None, role: str = "user", return_tensors: Optional[str] = "pt"):
        ids = self.get_prefix_tokens() + self._to_ids(self.build_prompt(query, history))
        row = {"input_ids": ids, "attention_mask": [1] * len(ids), "position_ids": list(range(len(ids)))}
        return self._tensors(type(self).pad(self, [row], padding=False), return_tensors)


@MindFormerRegister.register(MindFormerModuleType.TOKENIZER)
class ChatGLM4Tokenizer(_GLMChatMixin, _TiktokenStyle):
    """GLM-4 tokenizer (reference ``models/glm2/glm4_tokenizer.py``): tiktoken-style byte-pair ranks in
    ``tokenizer.model``, the role tokens (``<|system|>``, ``<|user|>``, ...) and ``build_chat_input`` /
    ``apply_chat_template`` with the ``[gMASK]<sop>`` prefix."""

    vocab_files_names = {"vocab_file": "tokenizer.model"}
    ROLE_TOKENS = ["<|endoftext|>", "[MASK]", "[gMASK]", "[sMASK]", "<sop>", "<eop>", "<|system|>", "<|user|>",
                   "<|assistant|>", "<|observation|>", "<|begin_of_image|>", "<|end_of_image|>",
                   "<|begin_of_video|>", "<|end_of_video|>"]

    def __init__(self, vocab_file: str, eos_token="<|endoftext|>", pad_token="<|endoftext|>", **kwargs):
        ranks = load_tiktoken_ranks(vocab_file)
        self._setup_bpe(ranks, {t: len(ranks) + i for i, t in enumerate(self.ROLE_TOKENS)})
        self.vocab_file = vocab_file
        kwargs.pop("add_bos_token", None)
        kwargs.pop("add_eos_token", None)
        super().__init__(vocab_file=vocab_file, eos_token=eos_token, pad_token=pad_token, **kwargs)

    def get_prefix_tokens(self) -> List[int]:
        return [self.get_command("[gMASK]"), self.get_command("<sop>")]


TOKENIZER_BY_MODEL_TYPE = {
    "llama": "LlamaTokenizer", "llama2": "LlamaTokenizer", "llama3": "Llama3Tokenizer", "llama3_1": "Llama3Tokenizer",
    "qwen2": "Qwen2Tokenizer", "qwen2_5": "Qwen2Tokenizer", "qwen3": "Qwen2Tokenizer", "qwen3_moe": "Qwen2Tokenizer",
    "chatglm2": "ChatGLM2Tokenizer", "glm2": "ChatGLM2Tokenizer", "chatglm": "ChatGLM3Tokenizer", "glm3": "ChatGLM3Tokenizer", "glm4": "ChatGLM4Tokenizer",
    "telechat": "TelechatTokenizer", "deepseek_v3": "LlamaTokenizerFast", "mixtral": "LlamaTokenizer",
}
TOKENIZER_CLASSES = {c.__name__: c for c in (LlamaTokenizer, LlamaTokenizerFast, Llama3Tokenizer, Qwen2Tokenizer,
                                             ChatGLM2Tokenizer, ChatGLM3Tokenizer, ChatGLM4Tokenizer, TelechatTokenizer)}
TOKENIZER_CLASSES["PreTrainedTokenizerFast"] = LlamaTokenizerFast
TOKENIZER_CLASSES["Qwen2TokenizerFast"] = LlamaTokenizerFast
