"""LoRA merge tool and the dataset preprocessing scripts."""
import json

import pytest
import torch

from mindformers_b200.models import ByteTokenizer, ChatGLM4Tokenizer
from mindformers_b200.models.tokenization_utils import save_tiktoken_ranks
from mindformers_b200.tools import transform_ckpt_lora as TL
from mindformers_b200.tools.dataset_preprocess.glm4 import alpaca_converter as glm_conv, glm4_preprocess
from mindformers_b200.tools.dataset_preprocess.llama import alpaca_converter, llama_preprocess
from mindformers_b200.tools.dataset_preprocess.llama.conversation import get_default_conv_template


def test_merge_lora_checkpoint(tmp_path):
    from safetensors.torch import load_file, save_file
    torch.manual_seed(0)
    w, a, b = torch.randn(6, 4), torch.randn(2, 4), torch.randn(6, 2)
    state = {"layers.0.attn.linear_proj.base.weight": w, "layers.0.attn.linear_proj.lora_a": a,
             "layers.0.attn.linear_proj.lora_b": b, "layers.0.norm.weight": torch.ones(4),
             "layers.1.mlp.fc.weight": w.clone(), "layers.1.mlp.fc.mindpet_delta_lora_a": a.clone(),
             "layers.1.mlp.fc.mindpet_delta_lora_b": b.clone()}
    (tmp_path / "src").mkdir()
    save_file(state, str(tmp_path / "src" / "ckpt.safetensors"))
    n = TL.main(["--src_ckpt_path_or_dir", str(tmp_path / "src"), "--dst_ckpt_dir", str(tmp_path / "dst"),
                 "--lora_scaling", "0.5"])
    assert n == 2
    out = load_file(str(tmp_path / "dst" / "checkpoint_0.safetensors"))
    assert set(out) == {"layers.0.attn.linear_proj.weight", "layers.0.norm.weight", "layers.1.mlp.fc.weight"}
    assert torch.allclose(out["layers.0.attn.linear_proj.weight"], w + 0.5 * b @ a, atol=1e-6)
    with pytest.raises(KeyError):
        TL.merge_lora_state({"x.lora_a": a}, 1.0)


def test_alpaca_and_llama_preprocess(tmp_path):
    recs = [{"instruction": "Add", "input": "1 2", "output": "3"}, {"instruction": "Hi", "input": "", "output": "hello"}]
    (tmp_path / "alpaca.json").write_text(json.dumps(recs))
    alpaca_converter.main(["--data_path", str(tmp_path / "alpaca.json"), "--output_path", str(tmp_path / "conv.json")])
    conv = json.loads((tmp_path / "conv.json").read_text())
    assert conv[0]["conversations"][0]["from"] == "human" and "### Input:\n1 2" in conv[0]["conversations"][0]["value"]
    assert conv[1]["conversations"][1] == {"from": "gpt", "value": "hello"}
    tok = ByteTokenizer()
    samples = llama_preprocess.tokenize_qa(tok, str(tmp_path / "conv.json"), seq_length=511)
    assert len(samples) == 2 and len(samples[0]["input_ids"]) == 512
    kept = [l for l in samples[1]["labels"] if l != -100]
    assert kept == tok.encode("hello", add_special_tokens=False) + [tok.eos_token_id]
    c = get_default_conv_template()
    c.append_message(c.roles[0], "hi")
    c.append_message(c.roles[1], None)
    assert c.get_prompt().endswith("USER: hi ASSISTANT:")
    (tmp_path / "wiki.tokens").write_text(" = Title = \n some text @-@ here , and more . \n" * 40)
    docs = llama_preprocess.tokenize_wiki(tok, [str(tmp_path / "wiki.tokens")], seq_length=63)
    assert docs and all(len(d) == 64 for d in docs)


def test_glm4_preprocess(tmp_path):
    recs = [{"instruction": "Translate", "input": "chat", "output": "cat"}]
    (tmp_path / "a.json").write_text(json.dumps(recs))
    glm_conv.main(["--data_path", str(tmp_path / "a.json"), "--output_path", str(tmp_path / "a.jsonl")])
    row = json.loads((tmp_path / "a.jsonl").read_text().splitlines()[0])
    assert row["messages"][0] == {"role": "user", "content": "Translate\nchat"}
    save_tiktoken_ranks({bytes([b]): b for b in range(256)}, str(tmp_path / "tokenizer.model"))
    n = glm4_preprocess.main(["--input_glob", str(tmp_path / "a.jsonl"), "--vocab_file", str(tmp_path / "tokenizer.model"),
                              "--seq_length", "64", "--output_file", str(tmp_path / "out" / "glm4")])
    assert n == 1
    sample = json.loads((tmp_path / "out" / "glm4.jsonl").read_text().splitlines()[0])
    tok = ChatGLM4Tokenizer(str(tmp_path / "tokenizer.model"))
    assert sample["input_ids"][:2] == tok.get_prefix_tokens() and len(sample["labels"]) == 64
    text = tok.decode([l for l in sample["labels"] if l != -100])
    assert "cat" in text and "Translate" not in text
