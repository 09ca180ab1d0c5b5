"""SFT / raw-text data loaders and the prompt-answer and multi-turn task datasets."""
import json

import pytest
import torch

from mindformers_b200.dataset import (ADGenDataLoader, KeyWordGenDataset, MultiSourceDataLoader, MultiTurnDataset,
                                      SFTDataLoader, ToolAlpacaDataLoader, TrainingDataLoader, read_records)
from mindformers_b200.models import ByteTokenizer, ChatGLM4Tokenizer
from mindformers_b200.models.tokenization_utils import save_tiktoken_ranks


def write_jsonl(path, rows):
    path.write_text("\n".join(json.dumps(r, ensure_ascii=False) for r in rows), encoding="utf-8")


def test_read_records_formats(tmp_path):
    rows = [{"a": "1", "b": "x"}, {"a": "2", "b": "y"}]
    write_jsonl(tmp_path / "d.jsonl", rows)
    (tmp_path / "d.json").write_text(json.dumps(rows))
    (tmp_path / "d.csv").write_text("a,b\n1,x\n2,y\n")
    (tmp_path / "d.tsv").write_text("a\tb\n1\tx\n2\ty\n")
    import pyarrow as pa
    import pyarrow.parquet as pq
    pq.write_table(pa.Table.from_pylist(rows), str(tmp_path / "d.parquet"))
    for name in ("d.jsonl", "d.json", "d.csv", "d.tsv", "d.parquet"):
        assert read_records(str(tmp_path / name)) == rows


def test_sft_alpaca_loader(tmp_path):
    write_jsonl(tmp_path / "alpaca.jsonl", [
        {"instruction": "Add", "input": "1 2", "output": "3"}, {"instruction": "Say hi", "input": "", "output": "hi"}])
    tok = ByteTokenizer()
    ds = SFTDataLoader(str(tmp_path), tok, dataset_name="alpaca", max_length=400)
    assert len(ds) == 2
    row = ds[0]
    assert row["input_ids"].shape == row["labels"].shape == (399,)
    kept = row["labels"][row["labels"] != -100].tolist()
    assert kept == tok.encode("3", add_special_tokens=False) + [tok.eos_token_id]
    # the label at position t is the input at t+1
    pos = (row["labels"] != -100).nonzero()[0].item()
    assert row["input_ids"][pos + 1].item() == row["labels"][pos].item()
    assert "### Input:" in tok.decode(row["input_ids"].tolist()) and "### Input:" not in tok.decode(ds[1]["input_ids"].tolist())
    assert row["loss_mask"].sum().item() == len(kept)


def test_sft_multi_round_chat(tmp_path):
    write_jsonl(tmp_path / "chat.jsonl", [{"conversations": [
        {"from": "human", "value": "hello"}, {"from": "gpt", "value": "hi!"},
        {"from": "human", "value": "bye"}, {"from": "gpt", "value": "ciao"}]}])
    tok = ByteTokenizer()
    ds = SFTDataLoader(str(tmp_path), tok, dataset_name="multi-round-chat", max_length=128, pad_to_max_length=False)
    row = ds[0]
    kept = row["labels"][row["labels"] != -100].tolist()
    e = lambda s: tok.encode(s, add_special_tokens=False)
    assert kept == e("hi!") + [tok.eos_token_id] + e("ciao") + [tok.eos_token_id]


def test_adgen_keyword_gen_dataset(tmp_path):
    write_jsonl(tmp_path / "train.json", [{"content": f"kw{i}", "summary": f"text {i}"} for i in range(6)])
    tok = ByteTokenizer(add_bos_token=False)
    rows = ADGenDataLoader(str(tmp_path / "train.json"), phase="train")
    assert rows[2] == {"prompt": "kw2", "answer": "text 2"}
    cfg = {"data_loader": {"type": "ADGenDataLoader", "dataset_dir": str(tmp_path / "train.json"), "phase": "train"},
           "tokenizer": tok, "max_source_length": 8, "max_target_length": 12, "batch_size": 2, "pin_memory": False}
    batches = list(KeyWordGenDataset(cfg))
    assert len(batches) == 3 and batches[0]["input_ids"].shape == (2, 19)
    lab = batches[0]["labels"][0]
    assert lab[lab != -100].tolist() == tok.encode("text 0", add_special_tokens=False) + [tok.eos_token_id]
    cfg["data_loader"]["phase"] = "eval"
    ev = next(iter(KeyWordGenDataset(cfg)))
    assert ev["input_ids"].shape == (2, 8) and ev["labels"].shape == (2, 12)
    assert ev["input_ids"][0, 0].item() == tok.pad_token_id and tok.decode(ev["input_ids"][0].tolist()) == "kw0"


def test_tool_alpaca_and_multi_turn(tmp_path):
    good = {"tools": [{"name": "weather"}], "conversations": [
        {"role": "user", "content": "weather in Paris?"},
        {"role": "tool", "name": "weather", "parameters": {"city": "Paris"}, "observation": {"temp": 20}},
        {"role": "assistant", "content": "20 degrees"}]}
    bad = {"conversations": [{"role": "assistant", "content": "?"}]}
    write_jsonl(tmp_path / "tool.jsonl", [good, bad])
    rows = ToolAlpacaDataLoader(str(tmp_path))
    assert len(rows) == 1 and rows.skipped == 1
    ranks = {bytes([b]): b for b in range(256)}
    save_tiktoken_ranks(ranks, str(tmp_path / "tokenizer.model"))
    tok = ChatGLM4Tokenizer(str(tmp_path / "tokenizer.model"))
    loader = MultiTurnDataset({"data_loader": rows, "tokenizer": tok, "max_seq_length": 512, "batch_size": 1,
                               "pin_memory": False})
    batch = next(iter(loader))
    ids, labels = batch["input_ids"][0], batch["labels"][0]
    assert ids.shape == labels.shape == (511,)
    assert ids[:2].tolist() == tok.get_prefix_tokens() and ids[2].item() == tok.get_command("<|system|>")
    text = tok.decode(labels[labels != -100].tolist())
    assert "tool_call(city='Paris')" in text and "20 degrees" in text and "weather in Paris" not in text
    assert '{"temp": 20}' not in text                      # observations carry no loss
    pos = (labels != -100).nonzero()[0].item()
    assert ids[pos + 1].item() == labels[pos].item()


def test_multi_source(tmp_path):
    write_jsonl(tmp_path / "a.jsonl", [{"content": f"a{i}", "summary": "x"} for i in range(4)])
    write_jsonl(tmp_path / "b.jsonl", [{"content": f"b{i}", "summary": "y"} for i in range(10)])
    subs = [{"type": "ADGenDataLoader", "dataset_dir": str(tmp_path / "a.jsonl")},
            {"type": "ADGenDataLoader", "dataset_dir": str(tmp_path / "b.jsonl")}]
    ds = MultiSourceDataLoader(subs)
    assert len(ds) == 14 and ds[0]["prompt"] == "a0" and ds[4]["prompt"] == "b0"
    ds = MultiSourceDataLoader(subs, dataset_ratios=[0.5, 0.5], samples_count=12, shuffle=True, seed=3)
    prompts = [ds[i]["prompt"] for i in range(len(ds))]
    assert len(prompts) == 12 and sum(p.startswith("a") for p in prompts) == 6
    assert prompts != sorted(prompts)
    again = MultiSourceDataLoader(subs, dataset_ratios=[0.5, 0.5], samples_count=12, shuffle=True, seed=3)
    assert prompts == [again[i]["prompt"] for i in range(12)]
    with pytest.raises(ValueError):
        MultiSourceDataLoader(subs, dataset_ratios=[0.5, 0.6])


def test_training_dataloader_packs_text(tmp_path):
    write_jsonl(tmp_path / "t.jsonl", [{"text": "abcdefghij"}, {"text": "klmnopqrst"}, {"text": "uvwxyz"}])
    tok = ByteTokenizer()
    ds = TrainingDataLoader(str(tmp_path), tok, max_length=9)
    samples = list(ds)
    stream = []
    for t in ("abcdefghij", "klmnopqrst", "uvwxyz"):
        stream += tok.encode(t, add_special_tokens=False) + [tok.eos_token_id]
    assert len(samples) == len(stream) // 9
    assert samples[0]["input_ids"].tolist() == stream[:8] and samples[0]["labels"].tolist() == stream[1:9]
    assert samples[1]["input_ids"].tolist() == stream[9:17]
    resumed = list(TrainingDataLoader(str(tmp_path), tok, max_length=9, skip_num=1))
    assert torch.equal(resumed[0]["input_ids"], samples[1]["input_ids"])
    assert len(list(TrainingDataLoader(str(tmp_path), tok, max_length=9, samples_num=2))) == 2


def test_hf_dataloader_with_handlers(tmp_path):
    from mindformers_b200.dataset.dataloaders import HFDataLoader
    write_jsonl(tmp_path / "alpaca.jsonl", [{"instruction": "Add", "input": "1 2", "output": "3"},
                                            {"instruction": "Say hi", "input": "", "output": "hi"}])
    tok = ByteTokenizer()
    ds = HFDataLoader(str(tmp_path / "alpaca.jsonl"), handler=[{"type": "AlpacaInstructDataHandler"}], tokenizer=tok,
                      seq_length=300)
    assert len(ds) == 2
    row = ds[1]
    assert row["input_ids"].shape == row["labels"].shape == (300,)
    kept = row["labels"][row["labels"] != -100].tolist()
    assert kept == tok.encode("hi", add_special_tokens=False) + [tok.eos_token_id]
    ds2 = HFDataLoader("json", data_files=str(tmp_path / "alpaca.jsonl"), handler=[{"type": "AlpacaInstructDataHandler"}],
                       tokenizer=tok, seq_length=300, num_samples=1)
    assert len(ds2) == 1
    import pytest as _pytest
    with _pytest.raises(FileNotFoundError):
        HFDataLoader("org/some_dataset")


def test_token_monitor_counts_what_the_loop_receives(tmp_path):
    import numpy as np
    import torch
    from mindformers_b200.dataset import CausalLanguageModelDataset
    loader = CausalLanguageModelDataset(dict(
        data_loader=dict(type="MockDataLoader", seq_length=16, vocab_size=50, num_samples=24, seed=3), batch_size=4,
        token_monitor=True, token_monitor_config=dict(vocab_size=50, dump_interval=2, save_dir=str(tmp_path))))
    seen = torch.zeros(50, dtype=torch.int64)
    for batch in loader:
        seen += torch.bincount(batch["input_ids"].reshape(-1), minlength=50)
    mon = loader.token_monitor
    assert torch.equal(mon.counts, seen) and mon.batches == 6
    s = mon.summary(top_k=3)
    assert s["tokens"] == int(seen.sum()) and len(s["top"]) == 3 and s["top"][0][1] == int(seen.max())
    assert np.load(tmp_path / "token_counts_rank0.npy").sum() == int(seen.sum())
