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


def test_moe_token_distribution_reports(tmp_path):
    import os
    """Expert-load dumps of a callback → merged tables, balance statistics and a chart per layer."""
    import json
    import numpy as np
    import torch
    from mindformers_b200.core.callback import RunContext, TopkBiasBalanceCallback
    from mindformers_b200.tools import moe_token_distribution_tools as tool

    class Router(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.expert_load = torch.zeros(8)

    model = torch.nn.Module()
    model.decoder = torch.nn.Module()
    model.decoder.layers = torch.nn.ModuleList([torch.nn.Module() for _ in range(3)])
    for i in (1, 2):
        model.decoder.layers[i].router = Router()

    class Engine:
        pass

    eng = Engine()
    eng.model = model
    cb = TopkBiasBalanceCallback(dump_dir=str(tmp_path / "dump"))
    for step in range(1, 6):
        model.decoder.layers[1].router.expert_load = torch.tensor([step, 1, 1, 1, 1, 1, 1, 0.0])    # expert 0 heats up
        model.decoder.layers[2].router.expert_load = torch.ones(8)
        cb.on_step_end(RunContext(engine=eng, global_step=step))
    files = tool.collect_npy_files(str(tmp_path / "dump"))
    assert sorted(files) == [1, 2] and len(files[1]) == 5 and files[1][0].endswith("layer-1-step1.npy")
    table = tool.merge_npy_files(files[1])
    assert table.shape == (5, 8) and table[4, 0] == 5
    reports = tool.generate_reports(str(tmp_path / "dump"), str(tmp_path / "charts") + "/", hot_expert_num=2)
    hot = reports[1]
    assert hot["hot_experts"][0] == 0 and hot["idle_experts"] == [7] and hot["cold_experts"][0] == 7
    assert hot["max_over_mean"]["last"] > hot["max_over_mean"]["first"] > 1.0
    even = reports[2]
    assert abs(even["max_over_mean"]["worst"] - 1.0) < 1e-9 and even["coefficient_of_variation"]["mean"] < 1e-9
    svg = open(tmp_path / "charts" / "layer-1.svg").read()
    assert svg.startswith("<svg") and svg.count("<rect") == 5 * 8
    assert json.load(open(tmp_path / "charts" / "layer-2.json"))["experts"] == 8
    assert np.loadtxt(tmp_path / "charts" / "layer-1.csv", delimiter=",").shape == (5, 8)
    tool.main(["--npy_files_load_path", str(tmp_path / "dump"), "--save_path_prefix", str(tmp_path / "c2") + "/",
               "--num_layers", "2"])
    assert os.path.exists(tmp_path / "c2" / "layer-1.svg") and not os.path.exists(tmp_path / "c2" / "layer-2.svg")


def test_deepseekv3_converter_streams_layers_and_handles_fp8(tmp_path):
    """Hugging Face style DeepSeek-V3 directory (several shards, one weight stored as block-scaled fp8 + scale_inv) →
    converter → framework directory that loads into the same model."""
    import importlib.util
    import json
    import os
    import torch
    from safetensors.torch import load_file, save_file
    from mindformers_b200.checkpoint.io import load_checkpoint, save_pretrained_dir
    from mindformers_b200.models import AutoModel
    from mindformers_b200.ops.functional import quantize_weight_128x128
    cfg = dict(model_type="deepseek_v3", num_hidden_layers=3, hidden_size=256, num_attention_heads=4,
               num_key_value_heads=4, intermediate_size=512, moe_intermediate_size=128, n_routed_experts=4,
               n_shared_experts=1, num_experts_per_tok=2, n_group=2, topk_group=1, routed_scaling_factor=1.0,
               norm_topk_prob=True, scoring_func="sigmoid", first_k_dense_replace=1, vocab_size=512, q_lora_rank=128,
               kv_lora_rank=128, qk_nope_head_dim=32, qk_rope_head_dim=16, v_head_dim=32, max_position_embeddings=128,
               params_dtype="float32", moe_router_enable_expert_bias=True)
    torch.manual_seed(3)
    src_model = AutoModel.from_config(cfg, device="cpu").eval()
    hf = tmp_path / "hf"
    save_pretrained_dir(src_model, str(hf), config_dict=cfg, max_shard_bytes=600_000, hf_names=True, family="deepseek_v3")
    assert len([f for f in os.listdir(hf) if f.endswith(".safetensors")]) > 3
    # store one projection the way the released checkpoint does: e4m3 values + one scale per 128 x 128 block
    key = "model.layers.1.self_attn.o_proj.weight"
    index = json.load(open(hf / "model.safetensors.index.json"))["weight_map"]
    shard = load_file(str(hf / index[key]))
    q, scale = quantize_weight_128x128(shard[key])
    shard[key], shard[key + "_scale_inv"] = q, scale
    save_file(shard, str(hf / index[key]), metadata={"format": "pt"})
    index[key + "_scale_inv"] = index[key]
    json.dump({"weight_map": index}, open(hf / "model.safetensors.index.json", "w"))
    spec = importlib.util.spec_from_file_location(
        "conv", os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "toolkit", "weight_convert",
                             "deepseekv3", "convert_deepseekv3_hf_weight.py"))
    conv = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(conv)
    out = conv.main(["--torch_ckpt_path", str(hf), "--mindspore_ckpt_path", str(tmp_path / "mf"), "--dtype", "fp32"])
    names = json.load(open(os.path.join(out, "model.safetensors.index.json")))["weight_map"]
    assert "decoder.layers.1.mlp.experts.weight1" in names and "decoder.layers.0.self_attention.linear_qkv.weight" in names
    dst_model = AutoModel.from_config(cfg, device="cpu").eval()
    load_checkpoint(dst_model, out, strict=True, family="deepseek_v3")
    a, b = dict(src_model.named_parameters()), dict(dst_model.named_parameters())
    for n in a:
        if n == "decoder.layers.1.self_attention.linear_proj.weight":
            rel = (a[n] - b[n]).norm() / a[n].norm()
            assert 0 < rel < 0.05                                   # went through e4m3
        else:
            assert torch.equal(a[n], b[n]), n


def test_fp8_cast_bf16_tool(tmp_path):
    import importlib.util
    import json
    import os
    import torch
    from safetensors.torch import load_file, save_file
    from mindformers_b200.ops.functional import quantize_weight_128x128
    src = tmp_path / "fp8"
    os.makedirs(src)
    torch.manual_seed(0)
    w = torch.randn(256, 128) * 0.1
    q, scale = quantize_weight_128x128(w)
    save_file({"a.weight": q, "norm.weight": torch.ones(8)}, str(src / "model-00001-of-00002.safetensors"))
    save_file({"a.weight_scale_inv": scale}, str(src / "model-00002-of-00002.safetensors"))      # scale in another shard
    json.dump({"model_type": "deepseek_v3", "quantization_config": {"fmt": "e4m3"}}, open(src / "config.json", "w"))
    spec = importlib.util.spec_from_file_location(
        "cast", os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "toolkit", "weight_convert",
                             "deepseekv3", "fp8_cast_bf16.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    dst = mod.main(["--input-fp8-hf-path", str(src), "--output-bf16-hf-path", str(tmp_path / "bf16")])
    out = load_file(os.path.join(dst, "model-00001-of-00002.safetensors"))
    assert out["a.weight"].dtype == torch.bfloat16 and (out["a.weight"].float() - w).norm() / w.norm() < 0.05
    idx = json.load(open(os.path.join(dst, "model.safetensors.index.json")))["weight_map"]
    assert set(idx) == {"a.weight", "norm.weight"}
    assert "quantization_config" not in json.load(open(os.path.join(dst, "config.json")))


def test_reference_package_name_aliases_the_implementation():
    import mindformers
    import mindformers.core.context as alias
    import mindformers_b200.core.context as real
    from mindformers import MindFormerConfig, Trainer                      # noqa: F401
    from mindformers.tools.register import MindFormerRegister
    from mindformers_b200.tools.register import MindFormerRegister as Real
    assert alias is real and MindFormerRegister is Real
    assert "Trainer" in dir(mindformers)


def test_version_map_and_automatic_pipeline_stages(monkeypatch):
    from mindformers_b200 import __version__
    from mindformers_b200.core.context import Context
    from mindformers_b200.run_check import MFCheck
    vm = MFCheck.version_map()
    assert __version__ in vm and "torch" in vm[__version__] and "sm_100a" in vm[__version__]["arch"]
    ctx = Context.__new__(Context)
    ctx.world_size, ctx.config = 32, {}
    monkeypatch.setenv("LOCAL_WORLD_SIZE", "8")                            # four servers of eight devices
    par = dict(model_parallel=2, pipeline_stage=1, micro_batch_num=8, data_parallel=16)
    assert ctx.choose_pipeline_stages(dict(par), auto=False) == 1
    p2 = dict(par)
    assert ctx.choose_pipeline_stages(p2, auto=True) == 4 and p2["data_parallel"] == 4
    assert ctx.choose_pipeline_stages(dict(par, micro_batch_num=2), auto=True) == 2     # never more stages than micro-batches


def test_benchmark_tools_resolve_models_prepare_data_and_train(tmp_path, monkeypatch):
    """``scripts/benchmark``: a preset name, a shipped configuration name and a model directory resolve; overrides
    reach the configuration; a raw text file and an Alpaca file are turned into datasets; weights in the model
    directory switch the run to fine-tuning."""
    import importlib.util
    import json as _json
    import os
    import shutil
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    bench_dir = os.path.join(root, "scripts", "benchmark")
    monkeypatch.syspath_prepend(bench_dir)

    def load(name):
        spec = importlib.util.spec_from_file_location(name, os.path.join(bench_dir, name + ".py"))
        mod = importlib.util.module_from_spec(spec)
        sys.modules[name] = mod
        spec.loader.exec_module(mod)
        return mod
    base = load("base_init_model")
    pre = load("run_pretrain")
    assert pre.build_args(["a=1", "b=0.5", "c=true", "d=none", "e=x"]) == {"a": 1, "b": 0.5, "c": True, "d": None, "e": "x"}
    named = base.BaseInitModel("llama3_1_8b", {"model_num_layers": 2, "data_seq_len": 256, "data_parallel": 1,
                                               "model_parallel": 1, "hidden_size": 128}, build_model=False)
    mc = named.config["model"]["model_config"]
    assert mc["num_hidden_layers"] == 2 and mc["seq_length"] == 256 and mc["hidden_size"] == 128 and named.custom_model
    assert named.config["parallel_config"]["model_parallel"] == 1 and not named.finetune
    with pytest.raises(ValueError):
        base.BaseInitModel("no_such_model", {}, build_model=False)
    # a model directory: yaml (+ later weights)
    mdir = tmp_path / "model"
    mdir.mkdir()
    shutil.copy(os.path.join(root, "configs", "general", "run_general_task.yaml"), mdir / "run.yaml")
    text = tmp_path / "wiki.train.tokens"
    text.write_text(" = Title = \n" + ("The quick brown fox jumps over the lazy dog . " * 400) + "\n")
    args = {"data_seq_len": 64, "data_batch_size": 2, "vocab_size": 300}
    run = pre.ModelPretrain(str(mdir), dict(args))
    assert not run.finetune
    res = run.train(str(text), steps=6, output_dir=str(tmp_path / "out"))
    assert res["mode"] == "train" and res["steps"] == 6 and res["tokens_per_s"] > 0 and res["final_loss"] < 6.0
    built = base.BaseInitModel(str(mdir), dict(args))
    assert built.network is not None and built.network.config.seq_length == 64
    # alpaca records, and weights in the directory -> fine-tuning
    alpaca = tmp_path / "alpaca_data.json"
    alpaca.write_text(_json.dumps([{"instruction": "add", "input": "1 2", "output": "3"},
                                   {"instruction": "say hi", "input": "", "output": "hi there"}] * 8))
    from mindformers_b200.checkpoint.io import save_checkpoint
    save_checkpoint(built.network, str(mdir / "weights.safetensors"))
    run2 = pre.ModelPretrain(str(mdir), dict(args))
    assert run2.finetune and run2.config["load_checkpoint"].endswith("weights.safetensors")
    res2 = run2.train(str(alpaca), steps=3, output_dir=str(tmp_path / "out2"))
    assert res2["mode"] == "finetune" and res2["steps"] == 3
    off = pre.ModelPretrain(str(mdir), dict(args, load_checkpoint=""))
    assert not off.finetune and off.config["load_checkpoint"] == ""


def test_multiprocess_safetensors_conversion_equals_the_single_process_one(tmp_path):
    """A Hugging Face directory whose shards cut a layer in two, converted by worker processes (the unit of work is a
    layer): same tensors as the single-process conversion, an index that names every tensor once, and the directory
    loads into a model."""
    import json
    import os
    import sys
    import torch
    from safetensors.torch import load_file, save_file
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import convert_weight
    from mindformers_b200.models import Qwen3MoeConfig, AutoModel, LlamaConfig, LlamaForCausalLM
    cfg = LlamaConfig(vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=5, num_attention_heads=4,
                      num_key_value_heads=2, params_dtype="float32", compute_dtype="float32")
    torch.manual_seed(0)
    m = LlamaForCausalLM(cfg, device="cpu")
    m.save_pretrained(str(tmp_path / "hf_one"), hf_names=True)
    full = {}
    for f in os.listdir(tmp_path / "hf_one"):
        if f.endswith(".safetensors"):
            full.update(load_file(str(tmp_path / "hf_one" / f)))
    keys = sorted(full)
    os.makedirs(tmp_path / "hf")
    cut = len(keys) // 3 + 1                                   # boundaries fall inside layers
    weight_map = {}
    for i in range(3):
        part = {k: full[k] for k in keys[i * cut:(i + 1) * cut]}
        save_file(part, str(tmp_path / "hf" / f"model-{i}.safetensors"))
        weight_map.update({k: f"model-{i}.safetensors" for k in part})
    json.dump({"weight_map": weight_map}, open(tmp_path / "hf" / "model.safetensors.index.json", "w"))
    json.dump(json.load(open(tmp_path / "hf_one" / "config.json")), open(tmp_path / "hf" / "config.json", "w"))
    single = load_file(convert_weight.main(["--model", "llama", "--input_path", str(tmp_path / "hf"),
                                            "--output_path", str(tmp_path / "one")]))
    index = convert_weight.main(["--model", "llama", "--input_path", str(tmp_path / "hf"), "--output_path",
                                 str(tmp_path / "many"), "--workers", "3"])
    wm = json.load(open(index))["weight_map"]
    assert len(set(wm.values())) >= 3 and set(wm) == set(single)
    merged = {}
    for f in set(wm.values()):
        merged.update(load_file(os.path.join(os.path.dirname(index), f)))
    assert all(torch.equal(merged[k], single[k]) for k in single)
    fresh = LlamaForCausalLM(cfg, device="cpu")
    from mindformers_b200.checkpoint.io import load_checkpoint
    load_checkpoint(fresh.model, os.path.dirname(index), strict=True)
    for (n, a), (_, b) in zip(m.model.named_parameters(), fresh.model.named_parameters()):
        assert torch.equal(a, b), n


def test_harness_adapter_serves_the_three_request_kinds(monkeypatch):
    """``MFLM`` under a stand-in for the lm-eval package (its ``TemplateLM`` base class and ``Instance`` requests): the
    adapter registers as model "mf", ``loglikelihood`` equals the summed log-probabilities of the continuation under
    the model, the greedy flag is right, rolling likelihoods add up over windows, ``generate_until`` cuts at the stop
    string, and a two-choice task scored from these numbers picks the likelier continuation."""
    import importlib
    import os
    import sys
    import types
    import torch
    registry = {}
    api = types.ModuleType("lm_eval.api")
    model_mod = types.ModuleType("lm_eval.api.model")
    reg_mod = types.ModuleType("lm_eval.api.registry")

    class TemplateLM:                                   # what the harness's base class provides
        def __init__(self):
            self.cache_hook = None

        def loglikelihood(self, requests, disable_tqdm=False):
            new = []
            for r in requests:
                context, continuation = r.args
                ctx = self.tok_encode(context) if context else [self.eot_token_id]
                new.append(((context, continuation), ctx, self.tok_encode(continuation)))
            return self._loglikelihood_tokens(new, disable_tqdm=disable_tqdm)

    model_mod.TemplateLM = TemplateLM
    reg_mod.register_model = lambda *names: (lambda cls: [registry.__setitem__(n, cls) for n in names] and cls)
    pkg = types.ModuleType("lm_eval")
    for name, mod in (("lm_eval", pkg), ("lm_eval.api", api), ("lm_eval.api.model", model_mod), ("lm_eval.api.registry", reg_mod)):
        monkeypatch.setitem(sys.modules, name, mod)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    monkeypatch.syspath_prepend(os.path.join(root, "toolkit", "benchmarks"))
    sys.modules.pop("eval_with_harness", None)
    ewh = importlib.import_module("eval_with_harness")
    assert registry.get("mf") is ewh.MFLM and issubclass(ewh.MFLM, TemplateLM)

    from mindformers_b200.models import ByteTokenizer, LlamaConfig, LlamaForCausalLM
    cfg = LlamaConfig(vocab_size=260, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, max_position_embeddings=128, seq_length=128, params_dtype="float32",
                      compute_dtype="float32", block_size=4)
    torch.manual_seed(0)
    model = LlamaForCausalLM(cfg, device="cpu")
    tok = ByteTokenizer()
    lm = ewh.MFLM(model=model, tokenizer=tok, max_length=64, max_gen_toks=8)

    class Instance:
        def __init__(self, *args):
            self.args = args

    ctx, a, b = "The capital of", " France", " Xq#z"
    (ll_a, g_a), (ll_b, g_b) = lm.loglikelihood([Instance(ctx, a), Instance(ctx, b)])
    ids = tok.encode(ctx, add_special_tokens=False) + tok.encode(a, add_special_tokens=False)
    with torch.no_grad():
        logp = torch.log_softmax(model.model(torch.tensor([ids])).float(), -1)
    n = len(tok.encode(a, add_special_tokens=False))
    want = sum(float(logp[i - 1, ids[i]]) for i in range(len(ids) - n, len(ids)))
    assert abs(ll_a - want) < 1e-4 and isinstance(g_a, bool)
    best = int(torch.tensor([ll_a, ll_b]).argmax())            # a two-choice task scored the harness way
    assert best == (0 if ll_a >= ll_b else 1)
    ctx_ids = tok.encode(ctx, add_special_tokens=False)
    greedy_ids = model.generate([ctx_ids], max_new_tokens=3, do_sample=False)[0][len(ctx_ids):]
    assert lm._loglikelihood_tokens([((ctx, ""), ctx_ids, greedy_ids)])[0][1] is True       # the model's own continuation
    assert lm._loglikelihood_tokens([((ctx, ""), ctx_ids, [(greedy_ids[0] + 1) % 256] + greedy_ids[1:])])[0][1] is False
    text = "abcdefghij" * 12                                    # longer than one window of 63 tokens
    rolling = lm.loglikelihood_rolling([Instance(text)])[0]
    short = lm.loglikelihood_rolling([Instance(text[:20])])[0]
    assert rolling < short < 0
    outs = lm.generate_until([Instance(ctx, {"until": ["\n"], "max_gen_toks": 6}), Instance(ctx, {"until": []})])
    assert len(outs) == 2 and all(isinstance(o, str) for o in outs) and "\n" not in outs[0]
    full = outs[1]
    if len(full) > 2:
        cut = lm.generate_until([Instance(ctx, {"until": [full[2]]})])[0]
        assert cut == full.split(full[2])[0]
