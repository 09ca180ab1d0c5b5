"""Entry points under ``research/``: packing of WikiText into an indexed dataset, flag handling of the shared predict
runner, per-family converter front ends."""
import importlib.util
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _load(rel):
    spec = importlib.util.spec_from_file_location(rel.replace("/", "_")[:-3], os.path.join(ROOT, rel))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_make_samples_stitch_and_pad():
    w = _load("research/deepseek3/wikitext_to_bin.py")
    docs = [[1, 2, 3], [4, 5], [6, 7, 8, 9]]
    stitched = list(w.make_samples(docs, 3, "stitch", eod=0, pad=-1, append_eod=False))
    assert stitched == [[1, 2, 3, 0], [4, 5, 0, 6], [7, 8, 9, 0]]
    padded = list(w.make_samples(docs, 3, "pad", eod=0, pad=99, append_eod=True))
    assert padded == [[1, 2, 3, 0], [4, 5, 0, 99], [6, 7, 8, 9]]


def test_wikitext_to_bin_writes_fixed_length_samples(tmp_path):
    from mindformers_b200.dataset.indexed_dataset import IndexedDataset
    w = _load("research/deepseek3/wikitext_to_bin.py")
    src = tmp_path / "wiki.tokens"
    src.write_text("\n = First = \n\n alpha beta gamma delta . \n\n = Second = \n\n one two three four five six . \n")
    prefix, n = w.main(["--input", str(src), "--output-prefix", str(tmp_path / "out" / "wiki"), "--tokenizer-type", "ByteTokenizer",
                        "--seq-length", "15"])
    ds = IndexedDataset(prefix)
    assert n >= 2 and len(ds) == n
    assert all(len(ds[i]) == 16 for i in range(n))
    from mindformers_b200.models import build_tokenizer
    tok = build_tokenizer({"type": "ByteTokenizer"})
    text = tok.decode([int(t) for i in range(n) for t in ds[i]])
    assert "alpha beta" in text and "one two" in text


def test_predict_runner_flags_and_overrides():
    from mindformers_b200.tools.register import MindFormerConfig
    r = _load("research/run_predict.py")
    args = r.build_parser().parse_args(["--yaml_file", "x.yaml", "--checkpoint_path", "ck", "--vocab_file_path", "v.model",
                                        "--max_length", "64", "--do_sample", "true", "--top_k", "3", "--use_past", "False",
                                        "--predict_data", "a", "b"])
    assert args.config == "x.yaml" and args.load_checkpoint == "ck" and args.vocab_file == "v.model" and args.predict_data == ["a", "b"]
    cfg = MindFormerConfig(model=dict(model_config=dict(seq_length=128, use_past=True)), processor=dict(tokenizer=dict(type="LlamaTokenizer")),
                           context=dict(device_id=0))
    r.apply_overrides(cfg, args)
    assert cfg.load_checkpoint == "ck" and cfg.processor.tokenizer.vocab_file == "v.model" and cfg.model.model_config.use_past is False
    assert cfg.generation.max_length == 64 and cfg.generation.do_sample is True and cfg.generation.top_k == 3 and cfg.run_mode == "predict"
    assert r.prompts_of(["x", ""]) == ["x"]
    with pytest.raises(SystemExit):
        r.main(["--predict_data", "hi"])           # no configuration


def test_family_converter_front_end(tmp_path, monkeypatch):
    import torch
    from safetensors.torch import load_file
    from mindformers_b200.models import LlamaConfig, LlamaForCausalLM
    c = _load("research/qwen2_5/convert_weight.py")
    seen = {}
    monkeypatch.setattr(c.convert_weight, "main", lambda argv: seen.setdefault("argv", argv))
    c.main(["--input_path", "a", "--output_path", "b"], reversed_=True)
    assert seen["argv"][:2] == ["--model", "qwen2_5"] and seen["argv"][-1] == "--reversed"


def test_research_aliases():
    import mindformers_b200 as mf
    assert _load("research/llama3_1/llama3_1_tokenizer.py").Llama3Tokenizer is mf.models.tokenizers.Llama3Tokenizer
    assert _load("research/llama3_1/llama.py").ParallelLlamaForCausalLM is mf.LlamaForCausalLM
    assert _load("research/qwen2_5/qwen2_5_tokenizer.py").Qwen2_5Tokenizer is mf.models.tokenizers.Qwen2Tokenizer
    assert _load("research/qwen2_5/run_qwen2_5.py").chatml("hi").endswith("<|im_start|>assistant\n")
