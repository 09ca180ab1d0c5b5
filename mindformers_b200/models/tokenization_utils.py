"""Tokenizer base class and the byte-level BPE engine shared by the concrete tokenizers.

``PreTrainedTokenizer`` covers what the reference's HF-derived base classes give a user
(``mindformers/models/tokenization_utils_base.py`` / ``tokenization_utils.py``): special-token bookkeeping, added
tokens that are split out before the model-specific ``_tokenize``, ``encode`` / ``decode`` / ``__call__`` with
padding, truncation and tensors, ``pad``, jinja2 chat templates, and ``save_pretrained`` / ``from_pretrained`` with
``tokenizer_config.json`` + ``special_tokens_map.json`` + the vocabulary files of the subclass. Subclasses implement
``_tokenize``, ``_convert_token_to_id``, ``_convert_id_to_token``, ``convert_tokens_to_string``, ``vocab_size`` and
``save_vocabulary``.

``BytePairEncoder`` is a rank-based byte-pair merger (the algorithm of tiktoken and of GPT-2 style ``merges.txt``
vocabularies): a piece of text is cut into bytes and the adjacent pair with the lowest rank is merged until none is
left. Both the Llama-3 / GLM-4 tiktoken files and the Qwen2 ``vocab.json`` + ``merges.txt`` pair load into it.
"""
from __future__ import annotations

import base64
import json
import os
from typing import Any, Dict, Iterable, List, Optional, Sequence, Tuple, Union

import regex as re

SPECIAL_TOKEN_ATTRIBUTES = ("bos_token", "eos_token", "unk_token", "sep_token", "pad_token", "cls_token", "mask_token")


class AddedToken:
    """A token that is matched in raw text before the model's own tokenisation."""

    def __init__(self, content: str, lstrip: bool = False, rstrip: bool = False, special: bool = False,
                 normalized: bool = False, single_word: bool = False):
        self.content, self.lstrip, self.rstrip = content, lstrip, rstrip
        self.special, self.normalized, self.single_word = special, normalized, single_word

    def __str__(self):
        return self.content

    def __repr__(self):
        return f"AddedToken({self.content!r}, special={self.special})"

    def __hash__(self):
        return hash(self.content)

    def __eq__(self, other):
        return str(self) == str(other)

    def to_dict(self):
        return {"content": self.content, "lstrip": self.lstrip, "rstrip": self.rstrip, "special": self.special,
                "normalized": self.normalized, "single_word": self.single_word}


class BatchEncoding(dict):
    """Dict of model inputs with attribute access and ``to(device)`` for tensor batches."""

    def __getattr__(self, item):
        try:
            return self[item]
        except KeyError as e:
            raise AttributeError(item) from e

    def to(self, device):
        for k, v in list(self.items()):
            if hasattr(v, "to"):
                self[k] = v.to(device)
        return self


class BytePairEncoder:
    """Rank-based byte-pair merging over ``bytes`` pieces.

    ``ranks`` maps a byte string to its rank, which is also its token id. ``pattern`` is the pre-tokenisation regex
    (``regex`` syntax). Merging keeps a list of parts and repeatedly joins the adjacent pair whose concatenation has
    the lowest rank; a small cache keeps whole pieces that were seen before.
    """

    def __init__(self, ranks: Dict[bytes, int], pattern: str):
        self.ranks = ranks
        self.pattern = re.compile(pattern)
        self.decoder = {v: k for k, v in ranks.items()}
        self._cache: Dict[bytes, List[int]] = {}

    def _merge(self, piece: bytes) -> List[int]:
        if piece in self.ranks:
            return [self.ranks[piece]]
        parts = [piece[i:i + 1] for i in range(len(piece))]
        while len(parts) > 1:
            best, best_rank = -1, None
            for i in range(len(parts) - 1):
                r = self.ranks.get(parts[i] + parts[i + 1])
                if r is not None and (best_rank is None or r < best_rank):
                    best, best_rank = i, r
            if best < 0:
                break
            parts[best:best + 2] = [parts[best] + parts[best + 1]]
        return [self.ranks[p] for p in parts]

    def encode_piece(self, piece: bytes) -> List[int]:
        ids = self._cache.get(piece)
        if ids is None:
            ids = self._merge(piece)
            if len(self._cache) < 65536:
                self._cache[piece] = ids
        return ids

    def encode_ordinary(self, text: str) -> List[int]:
        out: List[int] = []
        for m in self.pattern.findall(text):
            out.extend(self.encode_piece(m.encode("utf-8")))
        return out

    def decode_bytes(self, ids: Iterable[int]) -> bytes:
        return b"".join(self.decoder[i] for i in ids if i in self.decoder)


def load_tiktoken_ranks(path: str) -> Dict[bytes, int]:
    """A tiktoken vocabulary file: one ``<base64 token> <rank>`` pair per line."""
    ranks: Dict[bytes, int] = {}
    with open(path, "rb") as f:
        for line in f:
            line = line.strip()
            if line:
                tok, rank = line.split()
                ranks[base64.b64decode(tok)] = int(rank)
    return ranks


def save_tiktoken_ranks(ranks: Dict[bytes, int], path: str) -> None:
    with open(path, "wb") as f:
        for tok, rank in sorted(ranks.items(), key=lambda kv: kv[1]):
            f.write(base64.b64encode(tok) + b" " + str(rank).encode() + b"\n")


def bytes_to_unicode() -> Dict[int, str]:
    """GPT-2's reversible byte→printable-character table used by ``vocab.json`` files."""
    keep = list(range(ord("!"), ord("~") + 1)) + list(range(0xA1, 0xAD)) + list(range(0xAE, 0x100))
    table, extra = {}, 0
    for b in range(256):
        if b in keep:
            table[b] = chr(b)
        else:
            table[b] = chr(256 + extra)
            extra += 1
    return table


def load_gpt2_ranks(vocab_file: str, merges_file: Optional[str] = None) -> Dict[bytes, int]:
    """``vocab.json`` (printable-character tokens → id) as a bytes→rank table.

    GPT-2 style vocabularies list tokens in merge order after the 256 byte tokens, so the id doubles as the merge
    rank; ``merges.txt`` is only consulted to check that every merge result is present.
    """
    with open(vocab_file, "r", encoding="utf-8") as f:
        vocab = json.load(f)
    inv = {c: b for b, c in bytes_to_unicode().items()}
    ranks: Dict[bytes, int] = {}
    for tok, idx in vocab.items():
        try:
            ranks[bytes(inv[c] for c in tok)] = idx
        except KeyError:
            continue                      # an added/special token written in clear text
    if merges_file and os.path.exists(merges_file):
        with open(merges_file, "r", encoding="utf-8") as f:
            for line in f:
                if line.startswith("#") or not line.strip():
                    continue
                a, b = line.split()
                merged = bytes(inv[c] for c in a + b)
                if merged not in ranks:
                    raise ValueError(f"merge result {a + b!r} of {merges_file} is missing from {vocab_file}")
    return ranks


class PreTrainedTokenizer:
    """Base class of the slow (python) tokenizers. See the module docstring."""

    vocab_files_names: Dict[str, str] = {}
    model_input_names: List[str] = ["input_ids", "attention_mask"]
    padding_side: str = "right"
    truncation_side: str = "right"

    def __init__(self, **kwargs):
        self.init_kwargs = dict(kwargs)
        self.added_tokens_encoder: Dict[str, int] = {}
        self.added_tokens_decoder: Dict[int, AddedToken] = {}
        self._special: Dict[str, Optional[Union[str, AddedToken]]] = {a: None for a in SPECIAL_TOKEN_ATTRIBUTES}
        self.additional_special_tokens: List[str] = []
        self.model_max_length = int(kwargs.pop("model_max_length", 1 << 30))
        self.padding_side = kwargs.pop("padding_side", self.padding_side)
        self.truncation_side = kwargs.pop("truncation_side", self.truncation_side)
        self.chat_template = kwargs.pop("chat_template", None)
        self.clean_up_tokenization_spaces = kwargs.pop("clean_up_tokenization_spaces", False)
        self.add_bos_token = kwargs.pop("add_bos_token", getattr(self, "add_bos_token", False))
        self.add_eos_token = kwargs.pop("add_eos_token", getattr(self, "add_eos_token", False))
        for attr in SPECIAL_TOKEN_ATTRIBUTES:
            if kwargs.get(attr) is not None:
                self._special[attr] = kwargs[attr]
        extra = kwargs.get("additional_special_tokens") or []
        self.additional_special_tokens = [str(t) for t in extra]
        self._split_re = None
        # special tokens the model vocabulary does not know become added tokens
        self.add_tokens([t for t in self.all_special_tokens if self._convert_token_to_id_or_none(t) is None],
                        special_tokens=True)

    # ---- subclass interface -----------------------------------------------------------------------
    @property
    def vocab_size(self) -> int:
        raise NotImplementedError

    def _tokenize(self, text: str, **kwargs) -> List[Any]:
        raise NotImplementedError

    def _convert_token_to_id(self, token) -> Optional[int]:
        raise NotImplementedError

    def _convert_id_to_token(self, index: int):
        raise NotImplementedError

    def convert_tokens_to_string(self, tokens: List[Any]) -> str:
        raise NotImplementedError

    def save_vocabulary(self, save_directory: str, filename_prefix: Optional[str] = None) -> Tuple[str, ...]:
        return ()

    def get_vocab(self) -> Dict[Any, int]:
        vocab = {self._convert_id_to_token(i): i for i in range(self.vocab_size)}
        vocab.update(self.added_tokens_encoder)
        return vocab

    # ---- special tokens ---------------------------------------------------------------------------
    def __getattr__(self, name):
        # bos_token / bos_token_id and friends
        sp = self.__dict__.get("_special")
        if sp is not None:
            if name in sp:
                v = sp[name]
                return None if v is None else str(v)
            if name.endswith("_id") and name[:-3] in sp:
                v = sp[name[:-3]]
                return None if v is None else self.convert_tokens_to_ids(str(v))
        raise AttributeError(f"{type(self).__name__} has no attribute {name!r}")

    def __setattr__(self, name, value):
        sp = self.__dict__.get("_special")
        if sp is not None and name in sp:
            sp[name] = value
            if value is not None and self._convert_token_to_id_or_none(str(value)) is None:
                self.add_tokens([value], special_tokens=True)
            return
        if sp is not None and name.endswith("_id") and name[:-3] in sp and not isinstance(
                getattr(type(self), name, None), property):
            sp[name[:-3]] = None if value is None else self.convert_ids_to_tokens(value)
            return
        object.__setattr__(self, name, value)

    @property
    def special_tokens_map(self) -> Dict[str, Union[str, List[str]]]:
        out: Dict[str, Union[str, List[str]]] = {k: str(v) for k, v in self._special.items() if v is not None}
        if self.additional_special_tokens:
            out["additional_special_tokens"] = list(self.additional_special_tokens)
        return out

    @property
    def all_special_tokens(self) -> List[str]:
        seen: List[str] = []
        for v in list(self._special.values()) + list(self.additional_special_tokens):
            if v is not None and str(v) not in seen:
                seen.append(str(v))
        return seen

    @property
    def all_special_ids(self) -> List[int]:
        return [i for i in (self._token_to_id(t) for t in self.all_special_tokens) if i is not None]

    def _convert_token_to_id_or_none(self, token) -> Optional[int]:
        try:
            idx = self._convert_token_to_id(token)
        except (KeyError, NotImplementedError, AttributeError):
            return None
        unk = self._special.get("unk_token")
        if idx is not None and unk is not None and str(token) != str(unk):
            try:
                if idx == self._convert_token_to_id(str(unk)):
                    return None
            except (KeyError, AttributeError):
                pass
        return idx

    def add_tokens(self, new_tokens: Union[str, AddedToken, Sequence[Union[str, AddedToken]]],
                   special_tokens: bool = False) -> int:
        if isinstance(new_tokens, (str, AddedToken)):
            new_tokens = [new_tokens]
        added = 0
        for tok in new_tokens:
            content = str(tok)
            if content in self.added_tokens_encoder or not content:
                continue
            if self._convert_token_to_id_or_none(content) is not None and not special_tokens:
                continue
            known = self._convert_token_to_id_or_none(content)
            idx = known if known is not None else self.vocab_size + sum(
                1 for i in self.added_tokens_decoder if i >= self.vocab_size)
            obj = tok if isinstance(tok, AddedToken) else AddedToken(content, special=special_tokens)
            obj.special = obj.special or special_tokens
            self.added_tokens_encoder[content] = idx
            self.added_tokens_decoder[idx] = obj
            added += 1
        self._split_re = None
        return added

    def add_special_tokens(self, special_tokens_dict: Dict[str, Union[str, AddedToken, List[str]]]) -> int:
        added = 0
        for key, value in special_tokens_dict.items():
            if key == "additional_special_tokens":
                for t in value:
                    if str(t) not in self.additional_special_tokens:
                        self.additional_special_tokens.append(str(t))
                added += self.add_tokens(list(value), special_tokens=True)
            elif key in self._special:
                self._special[key] = value
                added += self.add_tokens([value], special_tokens=True)
            else:
                raise KeyError(f"{key} is not a special-token attribute")
        return added

    def __len__(self):
        return self.vocab_size + sum(1 for i in self.added_tokens_decoder if i >= self.vocab_size)

    # ---- text -> tokens -> ids --------------------------------------------------------------------
    def _splitter(self):
        if self._split_re is None and self.added_tokens_encoder:
            toks = sorted(self.added_tokens_encoder, key=len, reverse=True)
            self._split_re = re.compile("(" + "|".join(re.escape(t) for t in toks) + ")")
        return self._split_re

    def prepare_for_tokenization(self, text: str, **kwargs) -> Tuple[str, dict]:
        return text, kwargs

    def tokenize(self, text: str, **kwargs) -> List[Any]:
        text, kwargs = self.prepare_for_tokenization(text, **kwargs)
        sp = self._splitter()
        if sp is None:
            return self._tokenize(text, **kwargs) if text else []
        out: List[Any] = []
        for i, part in enumerate(sp.split(text)):
            if not part:
                continue
            if i % 2 == 1:
                out.append(part)
            else:
                out.extend(self._tokenize(part, **kwargs))
        return out

    def _token_to_id(self, token) -> Optional[int]:
        if isinstance(token, str) and token in self.added_tokens_encoder:
            return self.added_tokens_encoder[token]
        idx = self._convert_token_to_id(token)
        return idx

    def convert_tokens_to_ids(self, tokens):
        if isinstance(tokens, (str, bytes)):
            return self._token_to_id(tokens)
        return [self._token_to_id(t) for t in tokens]

    def convert_ids_to_tokens(self, ids, skip_special_tokens: bool = False):
        single = isinstance(ids, int)
        special = set(self.all_special_ids) if skip_special_tokens else ()
        out = []
        for i in ([ids] if single else ids):
            i = int(i)
            if i in special:
                continue
            out.append(self.added_tokens_decoder[i].content if i in self.added_tokens_decoder
                       else self._convert_id_to_token(i))
        return out[0] if single and out else out

    def num_special_tokens_to_add(self, pair: bool = False) -> int:
        return len(self.build_inputs_with_special_tokens([], [] if pair else None))

    def build_inputs_with_special_tokens(self, token_ids_0: List[int], token_ids_1: Optional[List[int]] = None):
        bos = [self.bos_token_id] if self.add_bos_token and self.bos_token_id is not None else []
        eos = [self.eos_token_id] if self.add_eos_token and self.eos_token_id is not None else []
        out = bos + list(token_ids_0) + eos
        if token_ids_1 is not None:
            out += bos + list(token_ids_1) + eos
        return out

    def get_special_tokens_mask(self, token_ids_0, token_ids_1=None, already_has_special_tokens: bool = False):
        if already_has_special_tokens:
            sp = set(self.all_special_ids)
            return [1 if t in sp else 0 for t in token_ids_0]
        b = 1 if self.add_bos_token and self.bos_token_id is not None else 0
        e = 1 if self.add_eos_token and self.eos_token_id is not None else 0
        mask = [1] * b + [0] * len(token_ids_0) + [1] * e
        if token_ids_1 is not None:
            mask += [1] * b + [0] * len(token_ids_1) + [1] * e
        return mask

    def create_token_type_ids_from_sequences(self, token_ids_0, token_ids_1=None):
        n0 = len(self.build_inputs_with_special_tokens(token_ids_0))
        if token_ids_1 is None:
            return [0] * n0
        return [0] * n0 + [1] * (len(self.build_inputs_with_special_tokens(token_ids_0, token_ids_1)) - n0)

    def encode(self, text: Union[str, List[int]], text_pair: Optional[Union[str, List[int]]] = None,
               add_special_tokens: bool = True, max_length: Optional[int] = None, truncation: bool = False,
               **kwargs) -> List[int]:
        ids0 = self._to_ids(text, **kwargs)
        ids1 = self._to_ids(text_pair, **kwargs) if text_pair is not None else None
        ids = self.build_inputs_with_special_tokens(ids0, ids1) if add_special_tokens else ids0 + (ids1 or [])
        if truncation and max_length is not None and len(ids) > max_length:
            ids = ids[:max_length] if self.truncation_side == "right" else ids[-max_length:]
        return ids

    def _to_ids(self, text, **kwargs) -> List[int]:
        if isinstance(text, str):
            return self.convert_tokens_to_ids(self.tokenize(text, **kwargs))
        if isinstance(text, (list, tuple)) and (not text or isinstance(text[0], int)):
            return list(text)
        if isinstance(text, (list, tuple)):
            return self.convert_tokens_to_ids(list(text))
        raise TypeError(f"cannot tokenise {type(text).__name__}")

    # ---- ids -> text ------------------------------------------------------------------------------
    def _decode(self, token_ids: List[int], skip_special_tokens: bool = False, **kwargs) -> str:
        special = set(self.all_special_ids) if skip_special_tokens else set()
        chunks: List[str] = []
        run: List[Any] = []
        for i in token_ids:
            i = int(i)
            if i in special:
                continue
            if i in self.added_tokens_decoder:
                if run:
                    chunks.append(self.convert_tokens_to_string(run))
                    run = []
                chunks.append(self.added_tokens_decoder[i].content)
            else:
                run.append(self._convert_id_to_token(i))
        if run:
            chunks.append(self.convert_tokens_to_string(run))
        return "".join(chunks)

    def decode(self, token_ids, skip_special_tokens: bool = False,
               clean_up_tokenization_spaces: Optional[bool] = None, **kwargs) -> str:
        if hasattr(token_ids, "tolist"):
            token_ids = token_ids.tolist()
        if isinstance(token_ids, int):
            token_ids = [token_ids]
        if token_ids and isinstance(token_ids[0], (list, tuple)):
            raise ValueError("decode takes one sequence; use batch_decode for a batch")
        text = self._decode(list(token_ids), skip_special_tokens=skip_special_tokens, **kwargs)
        clean = self.clean_up_tokenization_spaces if clean_up_tokenization_spaces is None else clean_up_tokenization_spaces
        if clean:
            for a, b in ((" .", "."), (" ?", "?"), (" !", "!"), (" ,", ","), (" n't", "n't"), (" 'm", "'m"),
                         (" 's", "'s"), (" 've", "'ve"), (" 're", "'re")):
                text = text.replace(a, b)
        return text

    def batch_decode(self, sequences, **kwargs) -> List[str]:
        if hasattr(sequences, "tolist"):
            sequences = sequences.tolist()
        return [self.decode(s, **kwargs) for s in sequences]

    # ---- batches ----------------------------------------------------------------------------------
    def _pad_one(self, enc: Dict[str, List[int]], width: int, side: str) -> Dict[str, List[int]]:
        n = len(enc["input_ids"])
        if "attention_mask" not in enc:
            enc["attention_mask"] = [1] * n
        gap = width - n
        if gap <= 0:
            return enc
        pad_id = self.pad_token_id if self.pad_token_id is not None else 0
        fill = {"input_ids": pad_id, "attention_mask": 0, "token_type_ids": 0, "special_tokens_mask": 1,
                "labels": -100, "position_ids": 0}
        for k in list(enc):
            if k in fill:
                pad = [fill[k]] * gap
                enc[k] = enc[k] + pad if side == "right" else pad + enc[k]
        return enc

    def pad(self, encoded_inputs, padding: Union[bool, str] = True, max_length: Optional[int] = None,
            pad_to_multiple_of: Optional[int] = None, return_tensors: Optional[str] = None,
            padding_side: Optional[str] = None) -> BatchEncoding:
        if isinstance(encoded_inputs, dict):
            first = encoded_inputs["input_ids"]
            if first and isinstance(first[0], (list, tuple)):
                rows = [{k: list(v[i]) for k, v in encoded_inputs.items()} for i in range(len(first))]
            else:
                rows = [{k: list(v) for k, v in encoded_inputs.items()}]
        else:
            rows = [{k: list(v) for k, v in e.items()} for e in encoded_inputs]
        width = None
        if padding in (True, "longest"):
            width = max(len(r["input_ids"]) for r in rows)
        elif padding == "max_length":
            width = max_length if max_length is not None else self.model_max_length
        if width is not None and pad_to_multiple_of:
            width = -(-width // pad_to_multiple_of) * pad_to_multiple_of
        side = padding_side or self.padding_side
        if width is not None:
            rows = [self._pad_one(r, width, side) for r in rows]
        out = BatchEncoding({k: [r[k] for r in rows] for k in rows[0]})
        return self._tensors(out, return_tensors)

    @staticmethod
    def _tensors(enc: BatchEncoding, return_tensors: Optional[str]) -> BatchEncoding:
        if return_tensors in (None, "list"):
            return enc
        if return_tensors == "pt":
            import torch
            return BatchEncoding({k: torch.tensor(v) for k, v in enc.items()})
        if return_tensors == "np":
            import numpy as np
            return BatchEncoding({k: np.asarray(v) for k, v in enc.items()})
        raise ValueError(f"return_tensors={return_tensors!r}: use 'pt', 'np' or None")

    def __call__(self, text, text_pair=None, add_special_tokens: bool = True, padding: Union[bool, str] = False,
                 truncation: bool = False, max_length: Optional[int] = None, return_tensors: Optional[str] = None,
                 return_attention_mask: bool = True, return_token_type_ids: bool = False,
                 return_special_tokens_mask: bool = False, pad_to_multiple_of: Optional[int] = None,
                 **kwargs) -> BatchEncoding:
        single = isinstance(text, str) or (isinstance(text, (list, tuple)) and text and isinstance(text[0], int))
        texts = [text] if single else list(text)
        pairs = [None] * len(texts) if text_pair is None else ([text_pair] if single else list(text_pair))
        rows = []
        for t, p in zip(texts, pairs):
            ids0 = self._to_ids(t, **kwargs)
            ids1 = self._to_ids(p, **kwargs) if p is not None else None
            ids = self.build_inputs_with_special_tokens(ids0, ids1) if add_special_tokens else ids0 + (ids1 or [])
            row = {"input_ids": ids}
            if return_token_type_ids:
                row["token_type_ids"] = (self.create_token_type_ids_from_sequences(ids0, ids1) if add_special_tokens
                                         else [0] * len(ids0) + [1] * len(ids1 or []))
            if return_special_tokens_mask:
                row["special_tokens_mask"] = (self.get_special_tokens_mask(ids0, ids1) if add_special_tokens
                                              else [0] * len(ids))
            if truncation and max_length is not None and len(ids) > max_length:
                cut = (lambda v: v[:max_length]) if self.truncation_side == "right" else (lambda v: v[-max_length:])
                row = {k: cut(v) for k, v in row.items()}
            if return_attention_mask:
                row["attention_mask"] = [1] * len(row["input_ids"])
            rows.append(row)
        if padding:
            enc = self.pad(rows, padding=padding, max_length=max_length, pad_to_multiple_of=pad_to_multiple_of)
        else:
            enc = BatchEncoding({k: [r[k] for r in rows] for k in rows[0]})
        if not return_attention_mask:
            enc.pop("attention_mask", None)
        if single and return_tensors is None:
            enc = BatchEncoding({k: v[0] for k, v in enc.items()})
        return self._tensors(enc, return_tensors)

    batch_encode_plus = __call__
    encode_plus = __call__

    # ---- chat templates ---------------------------------------------------------------------------
    default_chat_template: Optional[str] = None

    def apply_chat_template(self, conversation: List[Dict[str, str]], chat_template: Optional[str] = None,
                            add_generation_prompt: bool = False, tokenize: bool = True, padding: bool = False,
                            truncation: bool = False, max_length: Optional[int] = None,
                            return_tensors: Optional[str] = None, **template_kwargs):
        """Render ``conversation`` (``[{"role", "content"}, …]``) with the jinja2 chat template
        (reference: ``tokenization_utils_base.py`` ``apply_chat_template``)."""
        template = chat_template or self.chat_template or self.default_chat_template
        if template is None:
            raise ValueError(f"{type(self).__name__} has no chat template; pass chat_template=")
        from jinja2.sandbox import ImmutableSandboxedEnvironment

        def raise_exception(msg):
            raise ValueError(msg)

        env = ImmutableSandboxedEnvironment(trim_blocks=True, lstrip_blocks=True)
        env.globals["raise_exception"] = raise_exception
        rendered = env.from_string(template).render(
            messages=conversation, add_generation_prompt=add_generation_prompt, **self.special_tokens_map,
            **template_kwargs)
        if not tokenize:
            return rendered
        enc = self(rendered, add_special_tokens=False, padding=padding, truncation=truncation, max_length=max_length,
                   return_tensors=return_tensors)
        return enc["input_ids"]

    # ---- persistence ------------------------------------------------------------------------------
    def save_pretrained(self, save_directory: str, filename_prefix: Optional[str] = None) -> Tuple[str, ...]:
        os.makedirs(save_directory, exist_ok=True)
        cfg = {k: v for k, v in self.init_kwargs.items()
               if isinstance(v, (str, int, float, bool, type(None), list, dict)) and k not in self.vocab_files_names}
        cfg.update({k: str(v) for k, v in self._special.items() if v is not None})
        cfg["additional_special_tokens"] = list(self.additional_special_tokens)
        cfg["tokenizer_class"] = type(self).__name__
        cfg["padding_side"] = self.padding_side
        cfg["add_bos_token"], cfg["add_eos_token"] = self.add_bos_token, self.add_eos_token
        if self.model_max_length < (1 << 30):
            cfg["model_max_length"] = self.model_max_length
        if self.chat_template:
            cfg["chat_template"] = self.chat_template
        cfg["added_tokens_decoder"] = {str(i): t.to_dict() for i, t in sorted(self.added_tokens_decoder.items())}
        prefix = f"{filename_prefix}-" if filename_prefix else ""
        cfg_path = os.path.join(save_directory, prefix + "tokenizer_config.json")
        with open(cfg_path, "w", encoding="utf-8") as f:
            json.dump(cfg, f, indent=2, ensure_ascii=False)
        map_path = os.path.join(save_directory, prefix + "special_tokens_map.json")
        with open(map_path, "w", encoding="utf-8") as f:
            json.dump(self.special_tokens_map, f, indent=2, ensure_ascii=False)
        return (cfg_path, map_path) + tuple(self.save_vocabulary(save_directory, filename_prefix))

    @classmethod
    def from_pretrained(cls, directory: str, **kwargs):
        """Load from a directory written by ``save_pretrained`` (or an HF model dir that has this class's vocabulary
        files); a path to a single vocabulary file also works for one-file tokenizers."""
        cfg: Dict[str, Any] = {}
        if os.path.isfile(directory):
            key = next(iter(cls.vocab_files_names), "vocab_file")
            return cls(**{key: directory}, **kwargs)
        cfg_path = os.path.join(directory, "tokenizer_config.json")
        if os.path.exists(cfg_path):
            with open(cfg_path, "r", encoding="utf-8") as f:
                cfg = json.load(f)
        cfg.pop("tokenizer_class", None)
        cfg.pop("auto_map", None)
        added = cfg.pop("added_tokens_decoder", {}) or {}
        for k, v in list(cfg.items()):              # HF writes special tokens as AddedToken dicts
            if isinstance(v, dict) and "content" in v:
                cfg[k] = v["content"]
        for key, fname in cls.vocab_files_names.items():
            path = os.path.join(directory, fname)
            if os.path.exists(path):
                cfg[key] = path
        cfg.update(kwargs)
        missing = [k for k in cls.vocab_files_names if k not in cfg and k in cls.required_vocab_files()]
        if missing:
            raise FileNotFoundError(f"{directory} lacks {[cls.vocab_files_names[k] for k in missing]} for {cls.__name__}")
        tok = cls(**cfg)
        for idx, spec in sorted(added.items(), key=lambda kv: int(kv[0])):
            content = spec["content"] if isinstance(spec, dict) else str(spec)
            if content not in tok.added_tokens_encoder and tok._convert_token_to_id_or_none(content) is None:
                tok.added_tokens_encoder[content] = int(idx)
                tok.added_tokens_decoder[int(idx)] = AddedToken(content, special=bool(
                    spec.get("special", False)) if isinstance(spec, dict) else False)
        tok._split_re = None
        return tok

    @classmethod
    def required_vocab_files(cls) -> List[str]:
        return list(cls.vocab_files_names)[:1]
