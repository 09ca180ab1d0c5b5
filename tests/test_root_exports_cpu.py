"""The root package resolves the public names of the reference's root package, and the small classes behind the names
that have no dedicated test elsewhere do what their reference counterparts do."""
import json
import math
import os

import pytest
import torch

import mindformers_b200 as mf

# The names the reference's ``mindformers/__init__.py`` imports explicitly (grouped as there).
ROOT_NAMES = """
Trainer TrainingArguments BaseTrainer CausalLanguageModelingTrainer MultiModalToTextGenerationTrainer
AutoConfig AutoModel AutoModelForCausalLM AutoModelForMaskGeneration AutoModelForPreTraining AutoModelWithLMHead
AutoProcessor AutoTokenizer AutoImageProcessor CONFIG_MAPPING CONFIG_MAPPING_NAMES IMAGE_PROCESSOR_MAPPING TOKENIZER_MAPPING
BaseAudioProcessor BaseConfig BaseImageProcessor BaseModel BaseProcessor ImageProcessingMixin PretrainedConfig PreTrainedModel
PreTrainedTokenizer PreTrainedTokenizerBase PreTrainedTokenizerFast ProcessorMixin
ChatGLM2Config ChatGLM2ForConditionalGeneration ChatGLM2Model ChatGLM2Tokenizer ChatGLM2WithPtuning2 ChatGLM3Tokenizer
ChatGLM4Tokenizer GLMProcessor LlamaConfig LlamaForCausalLM LlamaModel LlamaProcessor LlamaTokenizer LlamaTokenizerFast
BaseDataset BaseMultiModalDataLoader CausalLanguageModelDataset KeyWordGenDataset MultiTurnDataset ModalToTextSFTDataset
check_dataset_config check_dataset_iterable build_dataset build_dataset_loader
MindFormerConfig DictConfig MindFormerRegister MindFormerModuleType ActionDict logger
TransformerOpParallelConfig EmbeddingOpParallelConfig OpParallelConfig TransformerRecomputeConfig MoEConfig
build_parallel_config reset_parallel_config build_context init_context
PetAdapter LoraAdapter PrefixTuningAdapter Ptuning2Adapter AdaAdapter AdaLoraAdapter LoraConfig PetConfig Ptuning2Config
PrefixTuningConfig
AlibiTensorV2 AttentionMaskHF RotaryEmbedding FixedSparseAttention LocalBlockSparseAttention Linear LayerNorm FreqsMgr
GenerationConfig GreedySearchLogitsProcessor LogitsProcessorList TopKLogitsWarper TopPLogitsWarper BaseStreamer TextStreamer
pipeline TextGenerationPipeline MultiModalToTextPipeline ModelRunner get_model
CrossEntropyLoss AdamW Came CheckpointMonitor MFLossMonitor EntityScore PerplexityMetric
MFTrainOneStepCell MFPipelineWithLossScaleCell
""".split()


@pytest.mark.parametrize("name", ROOT_NAMES)
def test_root_name_resolves(name):
    assert getattr(mf, name) is not None


def test_unknown_root_name_raises():
    with pytest.raises(AttributeError):
        mf.this_name_does_not_exist


def test_alibi_tensor_v2_matches_distance_times_slope():
    mod = mf.AlibiTensorV2(num_heads=6)
    mask = torch.tensor([[0, 0, 1, 1, 1], [1, 1, 1, 1, 0]])
    out = mod(mask)
    assert out.shape == (2, 6, 1, 5)
    # reference slopes: powers of 2^(-8/4) for the closest power of two (4), then odd powers of 2^(-8/8)
    slopes = [2 ** (-2.0 * (i + 1)) for i in range(4)] + [2 ** (-1.0 * (i + 1)) for i in (0, 2)]
    assert torch.allclose(mod.slopes, torch.tensor(slopes))
    assert torch.allclose(out[0, 1, 0], slopes[1] * torch.tensor([0.0, 0.0, 0.0, 1.0, 2.0]))
    assert torch.allclose(out[1, 5, 0], slopes[5] * torch.tensor([0.0, 1.0, 2.0, 3.0, 0.0]))


def test_attention_mask_hf_is_causal_and_respects_padding():
    m = mf.AttentionMaskHF(seq_length=4)(torch.tensor([[1, 1, 1, 0]]))
    want = torch.tensor([[[1, 0, 0, 0], [1, 1, 0, 0], [1, 1, 1, 0], [0, 0, 0, 0]]], dtype=torch.float32)
    assert torch.equal(m, want)


def test_legacy_rotary_embedding_rotates_halves():
    S, D = 5, 8
    inv = 1.0 / (10000 ** (torch.arange(0, D, 2).float() / D))
    ang = torch.outer(torch.arange(S).float(), inv)
    cos, sin = torch.cat([ang.cos()] * 2, -1), torch.cat([ang.sin()] * 2, -1)
    q, k = torch.randn(2, 3, S, D), torch.randn(2, 3, S, D)
    rq, rk = mf.RotaryEmbedding(head_dim=D)(q, k, (cos, sin, None))
    # rotation keeps the norm of every (i, i + D/2) pair and position 0 is the identity
    assert torch.allclose(rq[:, :, 0], q[:, :, 0], atol=1e-6) and torch.allclose(rk[:, :, 0], k[:, :, 0], atol=1e-6)
    assert torch.allclose(rq.norm(dim=-1), q.norm(dim=-1), atol=1e-5)
    # relative property: <R_m q, R_n k> depends on m - n only
    a = (rq[0, 0, 3] * rk[0, 0, 1]).sum()
    q2, k2 = q.roll(1, dims=2), k.roll(1, dims=2)
    rq2, rk2 = mf.RotaryEmbedding(head_dim=D)(q2, k2, (cos, sin, None))
    assert torch.allclose(a, (rq2[0, 0, 4] * rk2[0, 0, 2]).sum(), atol=1e-5)


def test_fixed_sparse_attention_pattern_and_values():
    B, S, H, D, blk, g = 2, 16, 2, 4, 8, 2
    layer = mf.FixedSparseAttention(num_heads=H, size_per_head=D, block_size=blk, seq_length=S, num_different_global_patterns=g)
    pat = layer.pattern
    assert pat.shape == (H, S, S) and not pat.triu(1).any()
    # query 12 (second block): own block causally, plus head 0 -> last half of block 0, head 1 -> first half
    assert pat[0, 12].nonzero().flatten().tolist() == [4, 5, 6, 7, 8, 9, 10, 11, 12]
    assert pat[1, 12].nonzero().flatten().tolist() == [0, 1, 2, 3, 8, 9, 10, 11, 12]
    q, k, v = (torch.randn(B, S, H * D) for _ in range(3))
    out = layer(q, k, v, torch.ones(B, S, S))
    qh, kh, vh = (t.view(B, S, H, D).transpose(1, 2) for t in (q, k, v))
    sc = (qh @ kh.transpose(-1, -2)) / math.sqrt(D)
    want = (torch.softmax(sc.masked_fill(~pat[None], float("-inf")), -1) @ vh).transpose(1, 2).reshape(B, S, H * D)
    assert torch.allclose(out, want, atol=1e-5)


def test_embedding_parallel_config_and_reset_parallel_config():
    e = mf.EmbeddingOpParallelConfig(data_parallel=2, model_parallel=4, vocab_emb_dp=False)
    assert e.dp_mp_config.model_parallel == 4 and e.to_dict()["vocab_emb_dp"] is False
    with pytest.raises(ValueError):
        mf.EmbeddingOpParallelConfig(model_parallel=0)
    with pytest.raises(TypeError):
        mf.EmbeddingOpParallelConfig(vocab_emb_dp=1)
    cfg = mf.MindFormerConfig(parallel_config=dict(data_parallel=2, model_parallel=2, micro_batch_num=4),
                              recompute_config=dict(recompute=True))
    built = mf.build_parallel_config(cfg)
    assert isinstance(cfg.parallel_config, mf.TransformerOpParallelConfig) and built.micro_batch_num == 4
    mf.reset_parallel_config(cfg)
    assert isinstance(cfg.parallel_config, dict) and cfg.parallel_config["micro_batch_num"] == 4
    assert "pipeline_stage" not in cfg.parallel_config          # defaults are dropped from the diff
    assert dict(cfg.recompute_config) == {"recompute": True}
    again = mf.build_parallel_config(cfg)
    assert again.data_parallel == 2 and again.recompute.recompute is True
    mf.reset_parallel_config(cfg, reset_diff_config=False)
    assert cfg.parallel_config["pipeline_stage"] == 1


def test_check_dataset_config_and_iterable():
    cfg = mf.MindFormerConfig(seed=7, profile=False, auto_tune=False, filepath_prefix="./autotune", autotune_per_step=10,
                              runner_config=dict(batch_size=4), parallel_config=dict(micro_batch_num=2),
                              train_dataset=dict(input_columns=["input_ids"], output_columns=None),
                              train_dataset_task=dict(type="CausalLanguageModelDataset"),
                              eval_dataset=dict(input_columns=["input_ids", "labels"]),
                              eval_dataset_task=dict(type="CausalLanguageModelDataset"))
    mf.check_dataset_config(cfg)
    tr, ev = cfg.train_dataset, cfg.eval_dataset
    assert tr.seed == 7 and tr.batch_size == 4 and tr.micro_batch_num == 2 and tr.do_eval is False
    assert tr.output_columns == ["input_ids"] and ev.do_eval is True and ev.output_columns == ["input_ids", "labels"]
    assert cfg.train_dataset_task.dataset_config is tr

    def gen():
        yield 1

    class Indexable:
        def __getitem__(self, i):
            return i

    assert mf.check_dataset_iterable([1, 2]) and mf.check_dataset_iterable(gen) and mf.check_dataset_iterable(Indexable())
    assert not mf.check_dataset_iterable(3) and not mf.check_dataset_iterable(len)
    dc = mf.BaseDataset.check_dataset_config(None, dict(dataset_config=None, batch_size=3, kwargs=dict(seed=1)))
    assert dc.batch_size == 3 and dc.seed == 1


def test_dict_config_attribute_access():
    d = mf.DictConfig(a=1, b=mf.DictConfig(c=2))
    assert d.a == 1 and d.b.c == 2 and d.missing is None
    d.e = 5
    assert d["e"] == 5 and d.to_dict() == {"a": 1, "b": {"c": 2}, "e": 5}
    del d.e
    assert "e" not in d


def test_base_multi_modal_dataloader(tmp_path):
    ann = tmp_path / "ann.json"
    ann.write_text(json.dumps([{"conversations": [{"from": "human", "value": "<image> what?"}, {"from": "gpt", "value": "a cat"}]},
                               {"conversations": [{"from": "human", "value": "hi"}, {"from": "gpt", "value": "hello"}]}]))
    rows = mf.BaseMultiModalDataLoader(str(ann), shuffle=False)
    assert len(rows) == 2 and rows[0]["conversations"] == [["human", "<image> what?"], ["gpt", "a cat"]]
    with pytest.raises(FileExistsError):
        mf.BaseMultiModalDataLoader(str(tmp_path / "none.json"))


def test_image_processor_save_and_auto_load(tmp_path):
    from mindformers_b200.models.multi_modal import BaseImageToTextImageProcessor

    class Proc(mf.ImageProcessingMixin, BaseImageToTextImageProcessor):
        pass

    mf.IMAGE_PROCESSOR_MAPPING.register("Proc", Proc, exist_ok=True)
    p = Proc(image_size=32, interpolation="bilinear")
    p.save_pretrained(str(tmp_path))
    saved = json.loads((tmp_path / "preprocessor_config.json").read_text())
    assert saved["image_processor_type"] == "Proc" and saved["image_size"] == 32
    q = mf.AutoImageProcessor.from_pretrained(str(tmp_path))
    assert isinstance(q, Proc) and q.image_size == 32 and q.interpolation == "bilinear"
    img = torch.rand(3, 40, 50)
    assert torch.allclose(p(img), q(img))
    assert isinstance(Proc.from_pretrained(str(tmp_path)), Proc)


def test_audio_processor_base_calls_preprocess():
    class Gain(mf.BaseAudioProcessor):
        def preprocess(self, audio_data, **kwargs):
            return [a * self.config["gain"] for a in audio_data]

    assert Gain(gain=2.0)([torch.ones(3)])[0].tolist() == [2.0, 2.0, 2.0]
    with pytest.raises(NotImplementedError):
        mf.BaseAudioProcessor()([1])


def test_auto_mappings():
    assert mf.CONFIG_MAPPING["llama"] is mf.LlamaConfig and "qwen3" in mf.CONFIG_MAPPING
    assert mf.CONFIG_MAPPING_NAMES["llama"] == "LlamaConfig"
    assert mf.TOKENIZER_MAPPING["llama"] is mf.LlamaTokenizer
    assert mf.AutoModelWithLMHead is mf.AutoModel and mf.AutoModelForPreTraining is mf.AutoModel


def _tiny(cls_cfg, **kw):
    return cls_cfg(vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
                   num_key_value_heads=2, max_position_embeddings=32, params_dtype="float32", compute_dtype="float32", **kw)


def test_llama_model_returns_hidden_states_consistent_with_lm_head():
    torch.manual_seed(0)
    cfg = _tiny(mf.LlamaConfig)
    backbone = mf.LlamaModel(cfg).eval()
    ids = torch.randint(0, 64, (2, 8))
    with torch.no_grad():
        hidden = backbone(ids)
        logits = mf.LlamaForCausalLM.forward(backbone, ids)
    assert hidden.shape == (16, 32)
    assert torch.allclose(backbone.model.logits(hidden).float(), logits, atol=1e-5)


def test_prefix_adapters_freeze_base_and_train_prefix():
    torch.manual_seed(0)
    model = mf.LlamaForCausalLM(_tiny(mf.LlamaConfig))
    tuned = mf.Ptuning2Adapter.get_pet_model(model, dict(pre_seq_len=4))
    trainable = [n for n, p in tuned.named_parameters() if p.requires_grad]
    assert trainable and all("prefix_encoder" in n for n in trainable)
    ids = torch.randint(0, 64, (2, 6))
    loss = tuned(ids, labels=ids)
    loss.backward()
    assert tuned.prefix_encoder.embedding.weight.grad.abs().sum() > 0
    k, v = torch.randn(2, 2, 6, 8), torch.randn(2, 2, 6, 8)
    pk, pv = torch.randn(2, 2, 4, 8), torch.randn(2, 2, 4, 8)
    k2, v2 = mf.Ptuning2Adapter.add_prefix((pk, pv), k, v)
    assert k2.shape == (2, 2, 10, 8) and torch.equal(k2[:, :, :4], pk) and torch.equal(v2[:, :, 4:], v)
    assert mf.Ptuning2Adapter.add_prefix(None, k, v)[0] is k
    with pytest.raises(NotImplementedError):
        mf.AdaLoraAdapter.get_pet_model(model, None)
    mf.PetAdapter.freeze_pretrained_model(model, "lora", freeze_exclude=["*final_layernorm*"])
    assert [n for n, p in model.named_parameters() if p.requires_grad] == [n for n, _ in model.named_parameters() if "final_layernorm" in n]


def test_chatglm2_with_ptuning2_trains_only_the_prefix():
    torch.manual_seed(0)
    cfg = mf.ChatGLM2Config(num_layers=2, padded_vocab_size=64, hidden_size=32, ffn_hidden_size=64, kv_channels=8,
                            num_attention_heads=4, multi_query_group_num=2, seq_length=32, params_dtype="float32",
                            compute_dtype="float32", pet_config=dict(pet_type="ptuning2", pre_seq_len=3))
    model = mf.ChatGLM2WithPtuning2(cfg)
    trainable = [n for n, p in model.named_parameters() if p.requires_grad]
    assert trainable and all(n.startswith("prefix_encoder") for n in trainable)
    ids = torch.randint(0, 64, (1, 5))
    model(ids, labels=ids).backward()
    assert model.prefix_encoder.embedding.weight.grad is not None


def test_chatglm2_tokenizer_prompt_rounds():
    prompt = mf.ChatGLM2Tokenizer.build_prompt(None, "q2", history=[("q1", "a1")])
    assert prompt == "[Round 1]\n\n问：q1\n\n答：a1\n\n[Round 2]\n\n问：q2\n\n答："


def test_get_model_returns_tokenizer_and_builder(tmp_path):
    with pytest.raises(ValueError):
        mf.get_model(str(tmp_path / "missing"))
    from tokenizers import Tokenizer, models, pre_tokenizers
    tok = Tokenizer(models.WordLevel({"<unk>": 0, "hello": 1, "world": 2, "<|user|>": 3, "<|assistant|>": 4}, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.Whitespace()
    tok.save(str(tmp_path / "tokenizer.json"))
    (tmp_path / "tokenizer_config.json").write_text(json.dumps({"tokenizer_class": "PreTrainedTokenizerFast", "unk_token": "<unk>"}))
    (tmp_path / "config.json").write_text(json.dumps({"model_type": "llama"}))
    tokenizer, builder = mf.get_model(str(tmp_path))
    assert tokenizer.encode("hello world")[-2:] == [1, 2]
    ids = builder.make_context(0, [{"role": "user", "content": "hello"}])
    assert 1 in ids


def _dense_attention(q, k, v, scale, discard=None, bias=None):
    rep = q.shape[1] // k.shape[1]
    s = (q.float() @ k.float().repeat_interleave(rep, 1).transpose(-1, -2)) * scale
    if bias is not None:
        s = s + bias
    if discard is not None:
        s = s.masked_fill(discard, float("-inf"))
    return torch.softmax(s, -1) @ v.float().repeat_interleave(rep, 1)


def test_flash_attention_layer_layouts_and_sparse_modes():
    from mindformers_b200.modules.flash_attention import FlashAttention
    torch.manual_seed(0)
    B, S, N, Nkv, D = 2, 12, 4, 2, 8
    q, k, v = torch.randn(B, N, S, D), torch.randn(B, Nkv, S, D), torch.randn(B, Nkv, S, D)
    scale = D ** -0.5
    causal = torch.triu(torch.ones(S, S, dtype=torch.bool), 1)
    want = _dense_attention(q, k, v, scale, causal)
    # BNSD, causal by sparse_mode
    out = FlashAttention(N, scale_value=scale, input_layout="BNSD", sparse_mode=2)(q, k, v)
    assert torch.allclose(out, want, atol=1e-5)
    # BSH, causal by an explicit mask (1 = discard)
    flat = lambda t: t.transpose(1, 2).reshape(B, S, -1)
    out = FlashAttention(N, scale_value=scale, input_layout="BSH", sparse_mode=0)(flat(q), flat(k), flat(v), causal.to(torch.uint8))
    assert torch.allclose(out, flat(want), atol=1e-5)
    # band: 3 tokens back, none ahead
    qi, ki = torch.arange(S)[:, None], torch.arange(S)[None, :]
    band = (ki > qi) | (ki < qi - 3)
    out = FlashAttention(N, scale_value=scale, input_layout="BNSD", sparse_mode=4, pre_tokens=3, next_tokens=0)(q, k, v)
    assert torch.allclose(out, _dense_attention(q, k, v, scale, band), atol=1e-5)
    # alibi bias
    bias = mf.AlibiTensorV2(N)(torch.ones(B, S))
    out = FlashAttention(N, scale_value=scale, input_layout="BNSD", sparse_mode=2, use_alibi_mask=True)(q, k, v, alibi_mask=bias)
    assert torch.allclose(out, _dense_attention(q, k, v, scale, causal, bias), atol=1e-5)
    # packed documents
    T = 10
    pq, pk, pv = torch.randn(T, N * D), torch.randn(T, Nkv * D), torch.randn(T, Nkv * D)
    out = FlashAttention(N, scale_value=scale, input_layout="TH", sparse_mode=3)(pq, pk, pv, actual_seq_qlen=[4, 10],
                                                                              actual_seq_kvlen=[4, 10])
    for a, b in ((0, 4), (4, 10)):
        qs = pq[a:b].view(1, b - a, N, D).transpose(1, 2)
        ks = pk[a:b].view(1, b - a, Nkv, D).transpose(1, 2)
        vs = pv[a:b].view(1, b - a, Nkv, D).transpose(1, 2)
        w = _dense_attention(qs, ks, vs, scale, torch.triu(torch.ones(b - a, b - a, dtype=torch.bool), 1))
        assert torch.allclose(out[a:b], w.transpose(1, 2).reshape(b - a, -1), atol=1e-5)


def test_la_pre_process_drops_padding_slots():
    import numpy as np
    from mindformers_b200.generation.parallel_decoding_mcore import compact_padded_tokens, la_pre_process
    slots = np.arange(12).reshape(3, 4)                # 3 sequences padded to 4 tokens
    out, mask = la_pre_process(None, slots, q_seq_lens=[2, 4, 1])
    assert out.tolist() == [0, 1, 4, 5, 6, 7, 8] and mask.shape == (1, 1)
    same, m2 = la_pre_process(None, np.arange(7), q_seq_lens=[2, 4, 1], spec_mask=np.ones((7, 7)))
    assert same.tolist() == list(range(7)) and m2.shape == (7, 7)
    assert la_pre_process(None, np.arange(3), q_seq_lens=1)[0].tolist() == [0, 1, 2]
    assert compact_padded_tokens(np.arange(12).reshape(3, 4) + 100, [2, 4, 1]).tolist() == [100, 101, 104, 105, 106, 107, 108]


def test_ckpt_transform_utils(tmp_path, capsys):
    from mindformers_b200.tools.ckpt_transform.utils import (check_ckpt_file_exist, check_path, check_rank_folders,
                                                             is_power_of_two, make_soft_link, show_progress)
    assert is_power_of_two(8) and not is_power_of_two(6) and not is_power_of_two(0)
    (tmp_path / "rank_0").mkdir()
    (tmp_path / "rank_0" / "a.safetensors").write_bytes(b"x")
    assert check_rank_folders(str(tmp_path), 0) and not check_rank_folders(str(tmp_path), 1)
    assert check_ckpt_file_exist(str(tmp_path / "rank_0")) and not check_ckpt_file_exist(str(tmp_path))
    link = tmp_path / "links" / "latest"
    make_soft_link(str(link), str(tmp_path / "rank_0"), target_is_directory=True)
    make_soft_link(str(link), str(tmp_path / "rank_0"), target_is_directory=True)        # replaces the link
    assert os.path.islink(link) and os.path.exists(link / "a.safetensors")
    with pytest.raises(FileNotFoundError):
        check_path(str(tmp_path / "nope"))
    show_progress(1.0, "transform")
    assert "100.00%" in capsys.readouterr().out
