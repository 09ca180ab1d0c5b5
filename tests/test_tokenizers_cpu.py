"""Tokenizers: the byte-pair engine against tiktoken, sentencepiece / tokenizers.json wrappers against their
libraries, padding / truncation / chat templates / save-load round trips."""
import json
import os

import pytest
import torch

from mindformers_b200.models import (AutoTokenizer, ChatGLM4Tokenizer, Llama3Tokenizer, LlamaTokenizer,
                                     LlamaTokenizerFast, Qwen2Tokenizer)
from mindformers_b200.models.tokenization_utils import (BytePairEncoder, bytes_to_unicode, load_tiktoken_ranks,
                                                        save_tiktoken_ranks)
from mindformers_b200.models.tokenizers import LLAMA3_PATTERN

CORPUS = ["the quick brown fox jumps over the lazy dog", "hello world, hello tokenizer!", "numbers 12345 and 678",
          "naïve café — ünïcödé", "def f(x):\n    return x + 1\n", "the the the and and over over"] * 4


def train_ranks(n_merges=120):
    """A small rank table by greedy pair counting over the corpus (bytes first, merges after)."""
    import regex as re
    pat = re.compile(LLAMA3_PATTERN)
    words = [[bytes([b]) for b in m.encode()] for line in CORPUS for m in pat.findall(line)]
    ranks = {bytes([b]): b for b in range(256)}
    for _ in range(n_merges):
        counts = {}
        for w in words:
            for a, b in zip(w, w[1:]):
                counts[(a, b)] = counts.get((a, b), 0) + 1
        if not counts:
            break
        (a, b), c = max(counts.items(), key=lambda kv: (kv[1], kv[0]))
        if c < 2:
            break
        ranks[a + b] = len(ranks)
        for w in words:
            i = 0
            while i < len(w) - 1:
                if w[i] == a and w[i + 1] == b:
                    w[i:i + 2] = [a + b]
                else:
                    i += 1
    return ranks


@pytest.fixture(scope="module")
def ranks():
    return train_ranks()


def test_bpe_matches_tiktoken(ranks):
    import tiktoken
    ref = tiktoken.Encoding("t", pat_str=LLAMA3_PATTERN, mergeable_ranks=ranks, special_tokens={})
    bpe = BytePairEncoder(ranks, LLAMA3_PATTERN)
    for text in CORPUS[:6] + ["over the lazy hello 42 ünï", "  leading spaces\n\n\ttabs"]:
        assert bpe.encode_ordinary(text) == ref.encode_ordinary(text)
        assert bpe.decode_bytes(bpe.encode_ordinary(text)).decode() == text


def test_llama3_tokenizer(tmp_path, ranks):
    path = str(tmp_path / "tokenizer.model")
    save_tiktoken_ranks(ranks, path)
    assert load_tiktoken_ranks(path) == ranks
    tok = Llama3Tokenizer(path)
    assert tok.vocab_size == len(ranks) + 256
    assert tok.bos_token_id == len(ranks) and tok.eos_token_id == len(ranks) + 1
    assert tok.convert_tokens_to_ids("<|eot_id|>") == len(ranks) + 9
    ids = tok.encode("hello world<|eot_id|>the fox")
    assert len(ranks) + 9 in ids
    assert tok.decode(ids) == "hello world<|eot_id|>the fox"
    assert tok.decode(ids, skip_special_tokens=True) == "hello worldthe fox"
    chat = tok.apply_chat_template([{"role": "user", "content": "hello"}], add_generation_prompt=True, tokenize=False)
    assert chat == ("<|begin_of_text|><|start_header_id|>user<|end_header_id|>\n\nhello<|eot_id|>"
                    "<|start_header_id|>assistant<|end_header_id|>\n\n")
    ids = tok.apply_chat_template([{"role": "user", "content": "hello"}], add_generation_prompt=True)
    assert ids[0] == tok.bos_token_id and tok.decode(ids) == chat
    # batch call: padding, truncation, tensors
    enc = tok(["hello world", "the quick brown fox jumps"], padding=True, return_tensors="pt")
    assert enc["input_ids"].shape == enc["attention_mask"].shape and enc["input_ids"].shape[0] == 2
    assert enc["attention_mask"][0].sum() < enc["attention_mask"][1].sum()
    assert (enc["input_ids"][0][enc["attention_mask"][0] == 0] == tok.pad_token_id).all()
    enc = tok("the quick brown fox jumps over", truncation=True, max_length=3)
    assert len(enc["input_ids"]) == 3
    enc = tok(["hello"], padding="max_length", max_length=8)
    assert len(enc["input_ids"][0]) == 8
    # save / load round trip through AutoTokenizer
    out = str(tmp_path / "saved")
    tok.save_pretrained(out)
    again = AutoTokenizer.from_pretrained(out)
    assert type(again).__name__ == "Llama3Tokenizer"
    assert again.encode("hello world<|eot_id|>") == tok.encode("hello world<|eot_id|>")


def test_added_tokens_and_padding_side(tmp_path, ranks):
    path = str(tmp_path / "tokenizer.model")
    save_tiktoken_ranks(ranks, path)
    tok = Llama3Tokenizer(path, padding_side="left")
    n = len(tok)
    assert tok.add_tokens(["<tool>", "</tool>"]) == 2 and len(tok) == n + 2
    ids = tok.encode("a<tool>b</tool>")
    assert n in ids and n + 1 in ids and tok.decode(ids) == "a<tool>b</tool>"
    tok.add_special_tokens({"additional_special_tokens": ["<extra>"]})
    assert tok.decode(tok.encode("x<extra>y"), skip_special_tokens=True) == "xy"
    enc = tok(["hello", "hello world the fox"], padding=True)
    assert enc["attention_mask"][0][0] == 0 and enc["attention_mask"][0][-1] == 1
    out = str(tmp_path / "saved")
    tok.save_pretrained(out)
    again = Llama3Tokenizer.from_pretrained(out)
    assert again.encode("a<tool>b</tool>") == ids and again.padding_side == "left"


def test_qwen2_tokenizer(tmp_path, ranks):
    table = bytes_to_unicode()
    vocab = {"".join(table[b] for b in tok): idx for tok, idx in ranks.items()}
    merges = ["#version: 0.2"]
    for tok_bytes, idx in sorted(ranks.items(), key=lambda kv: kv[1]):
        if len(tok_bytes) > 1:
            # find the split whose halves are both tokens of lower rank
            for cut in range(1, len(tok_bytes)):
                a, b = tok_bytes[:cut], tok_bytes[cut:]
                if a in ranks and b in ranks and ranks[a] < idx and ranks[b] < idx:
                    merges.append("".join(table[x] for x in a) + " " + "".join(table[x] for x in b))
                    break
    (tmp_path / "vocab.json").write_text(json.dumps(vocab), encoding="utf-8")
    (tmp_path / "merges.txt").write_text("\n".join(merges), encoding="utf-8")
    tok = Qwen2Tokenizer(str(tmp_path / "vocab.json"), str(tmp_path / "merges.txt"))
    base = len(ranks)
    assert (tok.end_of_text_id, tok.im_start_id, tok.im_end_id) == (base, base + 1, base + 2)
    assert tok.pad_token_id == base and tok.eos_token == "<|endoftext|>"
    text = "<|im_start|>user\nhello world<|im_end|>\n"
    ids = tok.encode(text)
    assert ids[0] == base + 1 and tok.decode(ids) == text
    prompt = tok.apply_chat_template([{"role": "user", "content": "hi"}], tokenize=False, add_generation_prompt=True)
    assert prompt.startswith("<|im_start|>system\nYou are a helpful assistant.<|im_end|>\n<|im_start|>user\nhi<|im_end|>")
    assert prompt.endswith("<|im_start|>assistant\n")
    out = tmp_path / "saved"
    tok.save_pretrained(str(out))
    again = AutoTokenizer.from_pretrained(str(out))
    assert isinstance(again, Qwen2Tokenizer) and again.encode(text) == ids


@pytest.fixture(scope="module")
def sp_model(tmp_path_factory):
    import sentencepiece as spm
    d = tmp_path_factory.mktemp("sp")
    corpus = d / "corpus.txt"
    corpus.write_text("\n".join(CORPUS * 8), encoding="utf-8")
    spm.SentencePieceTrainer.Train(input=str(corpus), model_prefix=str(d / "tokenizer"), vocab_size=360,
                                   model_type="bpe", character_coverage=1.0, byte_fallback=True,
                                   unk_id=0, bos_id=1, eos_id=2, pad_id=-1, minloglevel=2)
    return str(d / "tokenizer.model")


def test_llama_sentencepiece_tokenizer(tmp_path, sp_model):
    import sentencepiece as spm
    ref = spm.SentencePieceProcessor()
    ref.Load(sp_model)
    tok = LlamaTokenizer(sp_model)
    text = "the quick brown fox"
    assert tok.encode(text) == [1] + ref.EncodeAsIds(text)
    assert tok.encode(text, add_special_tokens=False) == ref.EncodeAsIds(text)
    assert tok.decode(tok.encode(text), skip_special_tokens=True) == text
    tok2 = LlamaTokenizer(sp_model, add_eos_token=True)
    assert tok2.encode(text)[-1] == 2
    pair = tok.encode("hello", "world")
    assert pair.count(1) == 2
    assert tok.get_special_tokens_mask(ref.EncodeAsIds(text))[0] == 1
    out = str(tmp_path / "saved")
    tok.save_pretrained(out)
    again = AutoTokenizer.from_pretrained(out)
    assert isinstance(again, LlamaTokenizer) and again.encode(text) == tok.encode(text)
    import pickle
    assert pickle.loads(pickle.dumps(tok)).encode(text) == tok.encode(text)


def test_fast_tokenizer_json(tmp_path):
    from tokenizers import Tokenizer, models, pre_tokenizers, decoders, trainers
    backend = Tokenizer(models.BPE(unk_token=None))
    backend.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    backend.decoder = decoders.ByteLevel()
    trainer = trainers.BpeTrainer(vocab_size=320, special_tokens=["<|begin|>", "<|end|>"], show_progress=False,
                                  initial_alphabet=pre_tokenizers.ByteLevel.alphabet())
    backend.train_from_iterator(CORPUS, trainer)
    path = str(tmp_path / "tokenizer.json")
    backend.save(path)
    tok = LlamaTokenizerFast(path, bos_token="<|begin|>", eos_token="<|end|>", pad_token="<|end|>", add_bos_token=True)
    text = "hello world, the fox"
    ids = tok.encode(text)
    assert ids[0] == tok.bos_token_id == backend.token_to_id("<|begin|>")
    assert ids[1:] == backend.encode(text, add_special_tokens=False).ids
    assert tok.decode(ids, skip_special_tokens=True) == text
    enc = tok([text, "hi"], padding=True, return_tensors="pt")
    assert isinstance(enc["input_ids"], torch.Tensor) and enc["input_ids"].shape[0] == 2
    n = tok.vocab_size
    assert tok.add_tokens(["<new_tok>"]) == 1 and tok.vocab_size == n + 1
    assert n in tok.encode("a<new_tok>b")
    out = str(tmp_path / "saved")
    tok.save_pretrained(out)
    again = AutoTokenizer.from_pretrained(out)
    assert isinstance(again, LlamaTokenizerFast) and again.encode(text) == ids


def test_glm4_chat_input(tmp_path, ranks):
    path = str(tmp_path / "tokenizer.model")
    save_tiktoken_ranks(ranks, path)
    tok = ChatGLM4Tokenizer(path)
    g, sop = tok.get_command("[gMASK]"), tok.get_command("<sop>")
    ids = tok.encode("hello")
    assert ids[:2] == [g, sop]
    enc = tok.build_chat_input("hello", history=[{"role": "system", "content": "be brief"}], return_tensors=None)
    row = enc["input_ids"][0]
    assert row[:2] == [g, sop] and row[2] == tok.get_command("<|system|>") and row[-1] == tok.get_command("<|assistant|>")
    assert tok.get_command("<|user|>") in row
    batch = tok(["hello", "hello world the quick fox"], padding=True)
    assert batch["attention_mask"][0][0] == 0                       # left padding
    assert batch["position_ids"][0][-1] == len([i for i in batch["attention_mask"][0] if i]) - 1


def test_processor_roundtrip(tmp_path, ranks):
    from mindformers_b200.models import AutoProcessor, LlamaProcessor, build_processor
    path = str(tmp_path / "tokenizer.model")
    save_tiktoken_ranks(ranks, path)
    tok = Llama3Tokenizer(path)
    proc = LlamaProcessor(tok, max_length=16)
    out = proc(text_input=["hello world", "the fox"])
    assert out["text"].shape == (2, 16) and out["attention_mask"].shape == (2, 16)
    proc.save_pretrained(str(tmp_path / "p"))
    again = AutoProcessor.from_pretrained(str(tmp_path / "p"))
    assert type(again).__name__ == "LlamaProcessor" and again.max_length == 16
    assert torch.equal(again(text_input=["hello world", "the fox"])["text"], out["text"])
    built = build_processor({"type": "LlamaProcessor", "tokenizer": {"type": "ByteTokenizer"}, "max_length": 8})
    assert built(text_input="abc")["text"].shape[-1] == 8


def test_slow_to_fast_conversion_encodes_alike(tmp_path, ranks):
    """``convert_slow_tokenizer``: the byte-level BPE tokenizers (Qwen2 and Llama-3 styles) rebuilt on the ``tokenizers``
    library give the same ids and round-trip the same texts, special tokens included; the merge list recovered from
    the rank table reproduces every multi-byte token."""
    from mindformers_b200.models import PreTrainedTokenizerFast, convert_slow_tokenizer
    from mindformers_b200.models.tokenizers import merges_from_ranks
    merges = merges_from_ranks(ranks)
    assert len(merges) == sum(len(t) > 1 for t in ranks) and all(a + b in ranks for a, b in merges)
    table = bytes_to_unicode()
    vocab = {"".join(table[b] for b in tok): idx for tok, idx in ranks.items()}
    (tmp_path / "vocab.json").write_text(json.dumps(vocab), encoding="utf-8")
    (tmp_path / "merges.txt").write_text("#version: 0.2\n" + "\n".join(
        "".join(table[x] for x in a) + " " + "".join(table[x] for x in b) for a, b in merges), encoding="utf-8")
    slow = Qwen2Tokenizer(str(tmp_path / "vocab.json"), str(tmp_path / "merges.txt"))
    fast = PreTrainedTokenizerFast(slow_tokenizer=slow)
    assert fast.vocab_size == slow.vocab_size and fast.eos_token == slow.eos_token
    texts = CORPUS[:7] + ["<|im_start|>user\nhello  world<|im_end|>\n", "tabs\tand\n\nnewlines   ", "数字 123 and ünï"]
    for t in texts:
        a, b = slow.encode(t), fast.encode(t)
        assert a == b, (t, a, b)
        assert fast.decode(b) == slow.decode(a) == t
    fast.save_pretrained(str(tmp_path / "fast"))
    again = AutoTokenizer.from_pretrained(str(tmp_path / "fast"))
    assert again.encode(texts[0]) == slow.encode(texts[0])
    backend = convert_slow_tokenizer(slow)
    assert backend.token_to_id("<|im_end|>") == slow.im_end_id
    with pytest.raises(TypeError):
        convert_slow_tokenizer(object())
