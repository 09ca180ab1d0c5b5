import numpy as np
import torch

from mindformers_b200.dataset import (BlendedDataset, CausalLanguageModelDataset, GPTDataset, GPTDatasetConfig,
                                      IndexedDataset, IndexedDatasetBuilder, MockGPTDataset, PackingHandler)
from mindformers_b200.dataset import helpers as H


def _oracle_sample_idx(sizes, doc_idx, seq, epochs, tokens_per_epoch, extra=1):
    """Flatten the documents, cut every seq tokens, and report (doc position, offset) of each cut."""
    starts, pos = [], 0
    for d in doc_idx:
        starts.append(pos)
        pos += sizes[d]
    n = (epochs * tokens_per_epoch - extra) // seq
    out = []
    for s in range(n + 1):
        tok = s * seq
        k = max(i for i, st in enumerate(starts) if st <= tok)
        # a cut that falls exactly on a document end stays in the previous document (offset = size - extra)
        if s > 0 and tok == starts[k] and k > 0 and extra == 1:
            pass
        out.append((k, tok - starts[k]))
    return out


def test_build_sample_idx_walks_the_token_stream():
    rng = np.random.RandomState(0)
    sizes = rng.randint(3, 40, size=20).astype(np.int32)
    doc_idx = np.concatenate([rng.permutation(20), rng.permutation(20)]).astype(np.int32)
    tpe = int(sizes.sum())
    got = H.build_sample_idx(sizes, doc_idx, 16, 2, tpe, True, 1)
    assert got.shape == ((2 * tpe - 1) // 16 + 1, 2)
    # every sample covers exactly seq+1 tokens of the flattened stream, consecutive samples overlap by one
    starts = np.concatenate(([0], np.cumsum(sizes[doc_idx])))[:-1]
    flat = starts[got[:, 0]] + got[:, 1]
    assert np.all(np.diff(flat) == 16)
    assert got[0].tolist() == [0, 0]


def test_blending_matches_weights_and_exhaustive_counts():
    di, ds = np.zeros(1000, np.int16), np.zeros(1000, np.int64)
    H.build_blending_indices(di, ds, [0.2, 0.5, 0.3], 3, 1000)
    assert abs((di == 0).mean() - 0.2) < 0.01 and abs((di == 1).mean() - 0.5) < 0.01
    for d in range(3):
        assert ds[di == d].tolist() == list(range(int((di == d).sum())))
    di, ds = np.zeros(12, np.int16), np.zeros(12, np.int64)
    H.build_exhaustive_blending_indices(di, ds, [2, 7, 3], 3)
    assert [(di == d).sum() for d in range(3)] == [2, 7, 3]


def test_build_mapping_rows_cover_documents():
    docs = np.array([0, 3, 5, 9])
    sizes = np.array([10, 12, 8, 30, 5, 7, 9, 11, 6], np.int32)
    rows = H.build_mapping(docs, sizes, 1, 100, 32, 0.0, 1234)
    assert sorted(rows[:, :2].tolist()) == [[0, 3], [3, 5], [5, 9]]
    blocks = H.build_blocks_mapping(docs, sizes, np.array([2, 2, 2], np.int32), 1, 100, 32, 1234)
    assert blocks.shape[1] == 4 and sorted(blocks[:, 2].tolist()) == [0, 1, 2]


def _make_indexed(tmp_path, n_docs=30, seed=0):
    rng = np.random.RandomState(seed)
    prefix = str(tmp_path / "corpus")
    b = IndexedDatasetBuilder(prefix + ".bin", dtype=np.uint16)
    docs = []
    for _ in range(n_docs):
        doc = rng.randint(1, 500, size=rng.randint(5, 60))
        docs.append(doc)
        b.add_item(doc)
        b.end_document()
    b.finalize(prefix + ".idx")
    return prefix, docs


def test_indexed_dataset_roundtrip_and_gpt_dataset(tmp_path):
    prefix, docs = _make_indexed(tmp_path)
    ds = IndexedDataset(prefix)
    assert len(ds) == len(docs)
    assert all(np.array_equal(ds[i], docs[i]) for i in range(len(docs)))
    assert ds.get(3, 2, 3).tolist() == docs[3][2:5].tolist()
    cfg = GPTDatasetConfig(sequence_length=32, random_seed=7, path_to_cache=str(tmp_path / "cache"))
    g = GPTDataset(ds, prefix, np.arange(len(ds), dtype=np.int32), 40, "train", cfg)
    assert len(g) >= 40
    item = g[5]
    assert item["input_ids"].shape == (32,) and torch.equal(item["input_ids"][1:], item["labels"][:-1])
    # cached indices are reused and give the same samples
    g2 = GPTDataset(ds, prefix, np.arange(len(ds), dtype=np.int32), 40, "train", cfg)
    assert torch.equal(g2[5]["input_ids"], item["input_ids"])


def test_mock_blend_loader_and_packing():
    cfg = GPTDatasetConfig(sequence_length=16, random_seed=1, vocab_size=100)
    a, b = MockGPTDataset(50, cfg, 100), MockGPTDataset(50, cfg, 100)
    assert torch.equal(a[3]["input_ids"], b[3]["input_ids"])
    blend = BlendedDataset([a, b], [0.25, 0.75], 40)
    assert len(blend) == 40 and int(blend[0]["dataset_id"]) in (0, 1)
    loader = CausalLanguageModelDataset({"data_loader": {"type": "MockDataLoader", "seq_length": 16, "vocab_size": 100,
                                                         "num_samples": 20}, "batch_size": 4, "pin_memory": False})
    batches = list(loader)
    assert len(batches) == 5 and batches[0]["input_ids"].shape == (4, 16)
    loader.set_init_step(3)
    assert len(list(loader)) == 2
    packed = PackingHandler(seq_length=16, max_segments=4).handle(
        [{"input_ids": np.arange(1, 8)}, {"input_ids": np.arange(1, 10)}, {"input_ids": np.arange(1, 6)}])
    assert len(packed) == 2 and packed[0]["actual_seq_len"].tolist() == [7, 16, 16, 16]


def test_indexed_dataset_from_an_object_store_prefix(tmp_path):
    import os
    """``s3://`` prefix: the index is cached locally once, token data comes from ranged reads (stand-in client)."""
    import numpy as np
    from mindformers_b200.dataset import IndexedDataset, IndexedDatasetBuilder
    from mindformers_b200.dataset.utils_s3 import S3Config
    prefix = str(tmp_path / "corpus")
    b = IndexedDatasetBuilder(prefix + ".bin", dtype=np.int32)
    docs = [np.arange(5), np.arange(100, 117), np.arange(7, 9)]
    for d in docs:
        b.add_item(d)
        b.end_document()
    b.finalize(prefix + ".idx")

    class FakeS3:
        def __init__(self):
            self.blobs = {("bkt", "data/corpus.idx"): open(prefix + ".idx", "rb").read(),
                          ("bkt", "data/corpus.bin"): open(prefix + ".bin", "rb").read()}

        def download_file(self, bucket, key, dst):
            open(dst, "wb").write(self.blobs[(bucket, key)])

        def get_object(self, Bucket, Key, Range):
            a, e = (int(x) for x in Range.split("=")[1].split("-"))
            return {"Body": self.blobs[(Bucket, Key)][a:e + 1]}

    ds = IndexedDataset("s3://bkt/data/corpus", object_storage_config=S3Config(str(tmp_path / "cache"), 64),
                        s3_client=FakeS3())
    assert len(ds) == 3
    for i, d in enumerate(docs):
        assert ds[i].tolist() == d.tolist()
    assert ds.get(1, offset=3, length=4).tolist() == [103, 104, 105, 106]
    assert ds._s3.requests <= 4 and os.path.exists(tmp_path / "cache" / "bkt" / "data" / "corpus.idx")


def test_pack_and_truncate_examples():
    from mindformers_b200.dataset.handler.packing_handler import PackingConfig, PackingHandler, pack_examples, truncate_examples
    cfg = PackingConfig(seq_length=8, pad_token=0, ignore_token=-100)
    samples = [{"input_ids": [1, 2, 3], "labels": [1, 2, 3]}, {"input_ids": [4, 5, 6, 7], "labels": [4, 5, 6, 7]},
               {"input_ids": [8, 9], "labels": [8, 9]}, {"input_ids": list(range(20, 30)), "labels": list(range(20, 30))}]
    packed = pack_examples(samples, cfg)
    # rows fill in order; the 10-token sample does not fit a row of 8 and is skipped
    assert packed["input_ids"] == [[1, 2, 3, 4, 5, 6, 7, 0], [8, 9, 0, 0, 0, 0, 0, 0]]
    assert packed["labels"][0] == [2, 3, 0, 5, 6, 7, 0, -100] and packed["actual_seq_len"] == [[3, 7], [2]]
    cols = {"input_ids": [[1, 2, 3], [4, 5, 6, 7], [8, 9, 10]], "labels": [[1, 2, 3], [4, 5, 6, 7], [8, 9, 10]]}
    cut = truncate_examples(cols, PackingConfig(seq_length=4))
    assert cut["input_ids"] == [[1, 2, 3, 4], [5, 6, 7, 8], [9, 10, 0, 0]]
    assert cut["labels"][-1] == [9, 10, -100, -100] and cut["actual_seq_len"] == [[3, 1], [3, 1], [2]]
    rows = PackingHandler(seq_length=4, pack_strategy="truncate", max_segments=4).handle(
        [{"input_ids": r, "labels": r} for r in cols["input_ids"]])
    assert [r["input_ids"].tolist() for r in rows] == cut["input_ids"]
    assert rows[0]["actual_seq_len"].tolist() == [3, 4, 4, 4] and rows[2]["actual_seq_len"].tolist() == [2, 4, 4, 4]
    with __import__("pytest").raises(ValueError):
        PackingConfig()


def test_indexed_dataset_dtype_codes_and_weight_split_helpers():
    import numpy as np
    import torch
    from mindformers_b200.dataset.indexed_dataset import DType
    from mindformers_b200.inference.weights_utils import (handle_training_ffn_weight, handle_training_qkv_weight,
                                                          split_weight_by_tp_rank)
    assert DType.code_from_dtype(np.int32) == 4 and DType.dtype_from_code(8) is np.uint16 and DType.size(5) == 8
    assert DType.optimal_dtype(32000) is np.uint16 and DType.optimal_dtype(152064) is np.int32
    w = torch.arange(24.).reshape(6, 4)
    assert torch.equal(split_weight_by_tp_rank(w, 0, 1, 2), w[3:]) and torch.equal(split_weight_by_tp_rank(w, 1, 0, 2), w[:, :2])

    class Cfg:
        num_attention_heads, num_query_groups, kv_channels, hidden_size = 4, 2, 2, 8

    q, k, v = torch.randn(8, 8), torch.randn(4, 8), torch.randn(4, 8)
    packed = torch.cat([torch.cat([q[g * 4:(g + 1) * 4], k[g * 2:(g + 1) * 2], v[g * 2:(g + 1) * 2]]) for g in range(2)])
    a, b, c = handle_training_qkv_weight(packed, Cfg)
    assert torch.equal(a, q) and torch.equal(b, k) and torch.equal(c, v)
    gate, up = handle_training_ffn_weight(torch.arange(12.).reshape(6, 2))
    assert gate.shape == (3, 2) and up[0, 0] == 6


def test_dynamic_length_sft_map_functions():
    from mindformers_b200.dataset.dataloader.sft_map_functions import (multi_instruct_dyn_map_fn, multi_round_chat_dyn_map_fn,
                                                                       multi_round_chat_dyn_map_fn_alpaca)

    class Tok:
        eos_token_id = 2

        def encode(self, text, add_special_tokens=False):
            return [10 + (ord(c) % 50) for c in text]

    tok = Tok()
    ex = {"conversations": [{"from": "human", "value": "hi"}, {"from": "gpt", "value": "yo"}]}
    row = multi_round_chat_dyn_map_fn(ex, tokenizer=tok, max_length=64, bos_token="", user_prompt_role="U:", assistant_prompt_role="A:")
    user = tok.encode("U:hi") + tok.encode("A:")
    assert row["input_ids"] == user + tok.encode("yo") + [2]
    assert row["labels"] == [-100] * len(user) + tok.encode("yo") + [2] and row["attention_mask"] == [1] * len(row["input_ids"])
    cut = multi_round_chat_dyn_map_fn(ex, tokenizer=tok, max_length=3, bos_token="")
    assert len(cut["input_ids"]) == 3 and len(cut["labels"]) == 3
    with __import__("pytest").raises(ValueError):
        multi_round_chat_dyn_map_fn({"conversations": [{"from": "bot", "value": "x"}]}, tokenizer=tok, max_length=8)
    ins = multi_instruct_dyn_map_fn({"instruction": "do ", "input": "x", "output": "ok"}, tokenizer=tok, max_length=64)
    assert ins["input_ids"] == tok.encode("do x") + tok.encode("ok") + [2] and ins["labels"][:4] == [-100] * 4
    al = multi_round_chat_dyn_map_fn_alpaca(ex, tokenizer=tok, max_length=256, bos_token="<s>", sep_token="|")
    assert al["input_ids"] == tok.encode("<s>|hi|") + tok.encode("yo<|im_end|>\n") + [2] and al["labels"] == al["input_ids"]
