"""CPU fp32 tests of the model stack, the optimizer and the parallel-state algebra."""
import copy

import pytest
import torch

from mindformers_b200.parallel.distributed.optimizer import DistributedOptimizer
from mindformers_b200.parallel.distributed.train_step import TrainOneStep
from mindformers_b200.parallel.layers.gpt_model import GPTModel
from mindformers_b200.parallel.parallel_state import RankGenerator
from mindformers_b200.parallel.transformer_config import MLATransformerConfig, TransformerConfig
from mindformers_b200.parallel.transformer_config_utils import convert_to_transformer_config


def tiny_llama_config(**kw):
    base = dict(num_layers=2, hidden_size=256, num_attention_heads=4, num_query_groups=2, ffn_hidden_size=688,
                vocab_size=1024, seq_length=128, max_position_embeddings=128, params_dtype="float32",
                compute_dtype="float32", use_scaled_init=False, layernorm_epsilon=1e-5, rotary_base=10000.0,
                pad_token_id=-1)
    base.update(kw)
    cfg = TransformerConfig(**base)
    cfg.device = "cpu"
    return cfg


def hf_llama_reference_loss(model, ids):
    """Independent re-statement of the tiny Llama forward in plain torch ops (fp32)."""
    cfg = model.config
    x = model.embedding.word_embeddings.weight[ids[:, :-1]]
    B, S, H = x.shape
    hd, nq, nkv = cfg.kv_channels, cfg.num_attention_heads, cfg.num_query_groups
    inv = 1.0 / (cfg.rotary_base ** (torch.arange(0, hd, 2).float() / hd))
    ang = torch.arange(S).float()[:, None] * inv[None]
    cos, sin = torch.cat((ang.cos(), ang.cos()), -1), torch.cat((ang.sin(), ang.sin()), -1)

    def rms(t, w):
        return t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + cfg.layernorm_epsilon) * w

    def rot(t):
        a, b = t[..., : hd // 2], t[..., hd // 2:]
        return torch.cat((-b, a), -1)

    for layer in model.decoder.layers:
        h = rms(x, layer.input_layernorm.weight)
        qkv = h @ layer.self_attention.linear_qkv.weight.t()
        q, k, v = qkv.split([nq * hd, nkv * hd, nkv * hd], -1)
        q = q.view(B, S, nq, hd)
        k = k.view(B, S, nkv, hd)
        v = v.view(B, S, nkv, hd)
        q = q * cos[None, :, None] + rot(q) * sin[None, :, None]
        k = k * cos[None, :, None] + rot(k) * sin[None, :, None]
        k = k.repeat_interleave(nq // nkv, 2)
        v = v.repeat_interleave(nq // nkv, 2)
        s = torch.einsum("bqhd,bkhd->bhqk", q, k) / hd ** 0.5
        s = s.masked_fill(torch.ones(S, S, dtype=torch.bool).triu(1), float("-inf"))
        o = torch.einsum("bhqk,bkhd->bqhd", s.softmax(-1), v).reshape(B, S, nq * hd)
        x = x + o @ layer.self_attention.linear_proj.weight.t()
        h = rms(x, layer.pre_mlp_layernorm.weight)
        gu = h @ layer.mlp.linear_fc1.weight.t()
        g, u = gu.chunk(2, -1)
        x = x + (torch.nn.functional.silu(g) * u) @ layer.mlp.linear_fc2.weight.t()
    x = rms(x, model.decoder.final_layernorm.weight)
    logits = x @ model.output_layer.weight.t()
    return torch.nn.functional.cross_entropy(logits.reshape(-1, logits.shape[-1]), ids[:, 1:].reshape(-1))


def test_tiny_llama_matches_independent_reference_and_adamw():
    torch.manual_seed(0)
    model = GPTModel(tiny_llama_config())
    assert sum(p.numel() for p in model.parameters()) == 1975552
    ids = torch.randint(0, 1024, (2, 129), generator=torch.Generator().manual_seed(3))
    loss = model(ids[:, :-1], ids[:, 1:])
    ref = hf_llama_reference_loss(model, ids)
    assert torch.allclose(loss, ref, atol=1e-5, rtol=1e-5)
    # one fwd + bwd + AdamW(lr 1e-4) step against torch.optim.AdamW on a deep copy
    twin = copy.deepcopy(model)
    opt = DistributedOptimizer(model, learning_rate=1e-4, betas=(0.9, 0.999), weight_decay=0.0, max_grad_norm=0.0)
    step = TrainOneStep(model, opt, micro_batch_size=2)
    out = step({"input_ids": ids[:, :-1].contiguous(), "labels": ids[:, 1:].contiguous()})
    topt = torch.optim.AdamW(twin.parameters(), lr=1e-4, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0)
    tl = twin(ids[:, :-1], ids[:, 1:])
    tl.backward()
    topt.step()
    assert abs(out["loss"].item() - tl.item()) < 1e-6
    for (n, a), (_, b) in zip(model.named_parameters(), twin.named_parameters()):
        assert torch.allclose(a, b, atol=1e-6), n


def test_training_is_bit_stable_across_runs():
    def run():
        torch.manual_seed(11)
        m = GPTModel(tiny_llama_config())
        opt = DistributedOptimizer(m, learning_rate=1e-3, max_grad_norm=1.0)
        step = TrainOneStep(m, opt, micro_batch_size=1)
        ids = torch.randint(0, 1024, (2, 65), generator=torch.Generator().manual_seed(5))
        losses = [step({"input_ids": ids[:, :-1].contiguous(), "labels": ids[:, 1:].contiguous()})["loss"].item()
                  for _ in range(3)]
        return losses, [p.detach().clone() for p in m.parameters()]

    l1, p1 = run()
    l2, p2 = run()
    assert l1 == l2 and l1[-1] < l1[0]
    assert all(torch.equal(a, b) for a, b in zip(p1, p2))


def test_gradient_accumulation_equals_large_batch():
    torch.manual_seed(2)
    a = GPTModel(tiny_llama_config())
    b = copy.deepcopy(a)
    ids = torch.randint(0, 1024, (4, 33))
    batch = {"input_ids": ids[:, :-1].contiguous(), "labels": ids[:, 1:].contiguous()}
    oa = DistributedOptimizer(a, learning_rate=1e-3)
    ob = DistributedOptimizer(b, learning_rate=1e-3)
    la = TrainOneStep(a, oa, micro_batch_size=4)(batch)["loss"]
    lb = TrainOneStep(b, ob, micro_batch_size=1)(batch)["loss"]
    assert abs(la.item() - lb.item()) < 1e-5
    ga, gb = oa.buffers["dense"].grad_data, ob.buffers["dense"].grad_data
    assert torch.allclose(ga, gb, atol=1e-6)
    assert abs(oa.global_norm().item() - ob.global_norm().item()) < 1e-5


def test_moe_mla_mtp_model_trains():
    torch.manual_seed(4)
    cfg = MLATransformerConfig(
        num_layers=3, hidden_size=128, num_attention_heads=4, ffn_hidden_size=256, vocab_size=512, seq_length=64,
        max_position_embeddings=64, params_dtype="float32", compute_dtype="float32", num_moe_experts=8,
        moe_router_topk=2, moe_ffn_hidden_size=64, first_k_dense_replace=1, moe_shared_expert_intermediate_size=64,
        q_lora_rank=32, kv_lora_rank=32, qk_head_dim=32, qk_pos_emb_head_dim=16, v_head_dim=32,
        moe_router_score_function="sigmoid", moe_router_enable_expert_bias=True, moe_aux_loss_coeff=1e-3,
        rotary_scaling_factor=1.0, mtp_num_layers=1, moe_router_num_groups=4, moe_router_group_topk=2,
        moe_router_topk_scaling_factor=2.5)
    cfg.device = "cpu"
    model = GPTModel(cfg)
    names = {n for n, _ in model.named_parameters()}
    for expect in ("decoder.layers.1.mlp.router.weight", "decoder.layers.1.mlp.experts.weight1",
                   "decoder.layers.1.mlp.shared_experts.linear_fc1.weight", "decoder.layers.0.mlp.linear_fc1.weight",
                   "decoder.layers.1.self_attention.linear_qb.weight", "decoder.layers.1.self_attention.linear_kvb.weight",
                   "mtp.layers.0.eh_proj.weight", "mtp.layers.0.enorm.weight", "decoder.final_layernorm.weight"):
        assert expect in names, expect
    opt = DistributedOptimizer(model, learning_rate=2e-3)
    step = TrainOneStep(model, opt, micro_batch_size=2)
    ids = torch.randint(0, 512, (2, 65))
    batch = {"input_ids": ids[:, :-1].contiguous(), "labels": ids[:, 1:].contiguous()}
    losses = [step(batch)["loss"].item() for _ in range(5)]
    assert losses[-1] < losses[0]
    model.update_topk_bias()
    bias = model.decoder.layers[1].mlp.router.expert_bias
    assert bias.abs().max() > 0


def test_moe_dispatch_matches_dense_loop():
    from mindformers_b200.parallel.layers.moe import MoELayer
    torch.manual_seed(6)
    cfg = tiny_llama_config(num_moe_experts=4, moe_router_topk=2, moe_ffn_hidden_size=64, hidden_size=64,
                            num_attention_heads=4, num_query_groups=4, ffn_hidden_size=128)
    layer = MoELayer(cfg)
    x = torch.randn(37, 64)
    out, _ = layer(x)
    probs, ids, _ = layer.router(x)
    ref = torch.zeros_like(x)
    for t in range(x.shape[0]):
        for j in range(2):
            e = ids[t, j].item()
            h = x[t] @ layer.experts.weight1[e]
            g, u = h.chunk(2)
            ref[t] += probs[t, j] * ((torch.nn.functional.silu(g) * u) @ layer.experts.weight2[e])
    assert torch.allclose(out, ref, atol=1e-5)


def test_rank_generator_groups_are_orthogonal():
    g = RankGenerator(tp=2, ep=1, dp=2, pp=2, cp=1)
    assert g.get_ranks("tp") == [[0, 1], [2, 3], [4, 5], [6, 7]]
    assert g.get_ranks("dp") == [[0, 2], [1, 3], [4, 6], [5, 7]]
    assert g.get_ranks("pp") == [[0, 4], [1, 5], [2, 6], [3, 7]]
    flat = sorted(r for grp in g.get_ranks("tp-dp") for r in grp)
    assert flat == list(range(8))
    e = RankGenerator(tp=1, ep=4, dp=2, pp=1, cp=1)
    assert e.get_ranks("ep") == [[0, 1, 2, 3], [4, 5, 6, 7]]


def test_hf_config_conversion():
    hf = dict(model_type="qwen3_moe", num_hidden_layers=4, hidden_size=64, num_attention_heads=4,
              num_key_value_heads=2, head_dim=16, intermediate_size=128, moe_intermediate_size=32, num_experts=8,
              num_experts_per_tok=2, vocab_size=100, rms_norm_eps=1e-6, rope_theta=1e6, norm_topk_prob=True,
              parallel_config=dict(model_parallel=1, expert_parallel=1, use_seq_parallel=False))
    cfg = convert_to_transformer_config(hf)
    assert cfg.num_layers == 4 and cfg.num_query_groups == 2 and cfg.kv_channels == 16
    assert cfg.num_moe_experts == 8 and cfg.moe_router_topk == 2 and cfg.moe_ffn_hidden_size == 32
    assert cfg.rotary_base == 1e6 and cfg.layernorm_epsilon == 1e-6
    with pytest.raises(KeyError):
        convert_to_transformer_config(dict(hf, num_layers=3))
    with pytest.raises(ValueError):
        convert_to_transformer_config(dict(hf, definitely_unknown_key=1))


def test_layer_specs_describe_and_drive_the_layers():
    """The decoder is built from layer specs: dense / MoE pattern, MLA switch, and a replaced sub-module class."""
    from mindformers_b200.parallel.layers.attention import MLASelfAttention, SelfAttention
    from mindformers_b200.parallel.layers.gpt_layer_specs import (get_gpt_decoder_block_spec, get_gpt_layer_local_spec,
                                                                  get_gpt_mtp_block_spec)
    from mindformers_b200.parallel.layers.mlp import MLP
    from mindformers_b200.parallel.layers.moe import MoELayer
    from mindformers_b200.parallel.layers.transformer_layer import TransformerLayer
    from mindformers_b200.parallel.spec_utils import ModuleSpec, build_module

    dense = get_gpt_layer_local_spec()
    assert dense.module is TransformerLayer and dense.submodules.self_attention.module is SelfAttention
    assert dense.submodules.mlp.module is MLP and dense.submodules.post_mlp_layernorm is None
    moe = get_gpt_layer_local_spec(num_experts=8, multi_latent_attention=True, sandwich_norm=True)
    assert moe.submodules.self_attention.module is MLASelfAttention and moe.submodules.mlp.module is MoELayer
    assert moe.submodules.post_attn_layernorm is not None

    cfg = tiny_llama_config(num_layers=3, num_moe_experts=4, moe_router_topk=2, moe_ffn_hidden_size=64,
                            first_k_dense_replace=1)
    specs = get_gpt_decoder_block_spec(cfg)
    assert [s.submodules.mlp.module is MoELayer for s in specs] == [False, True, True]
    assert get_gpt_mtp_block_spec(cfg) is None
    model = GPTModel(cfg)
    assert [layer.is_moe for layer in model.decoder.layers] == [False, True, True]

    class TaggedAttention(SelfAttention):
        pass

    spec = get_gpt_layer_local_spec()
    spec.submodules.self_attention = ModuleSpec(module=TaggedAttention)
    layer = build_module(spec, tiny_llama_config(), layer_number=1)
    assert type(layer.self_attention) is TaggedAttention and not layer.is_moe
    assert set(dict(layer.named_parameters())) == set(dict(TransformerLayer(tiny_llama_config()).named_parameters()))


def test_unfused_attention_path_and_masks():
    """``use_flash_attention=False`` goes through mask generation + scale-mask-softmax and gives the same loss; the
    mask generator separates documents after a position reset and by cumulative segment ends."""
    from mindformers_b200.parallel.layers.dot_product_attention import (CausalMaskGenerate, DotProductAttention,
                                                                        FusedScaleMaskSoftmax, LowerTriangularMask)
    torch.manual_seed(3)
    ids = torch.randint(0, 1024, (2, 33))
    a = GPTModel(tiny_llama_config())
    b = GPTModel(tiny_llama_config(use_flash_attention=False))
    b.load_state_dict(a.state_dict())
    assert isinstance(b.decoder.layers[0].self_attention.core_attention.unfused, DotProductAttention)
    la = a(ids[:, :-1].contiguous(), labels=ids[:, 1:].contiguous())
    lb = b(ids[:, :-1].contiguous(), labels=ids[:, 1:].contiguous())
    assert abs(float(la.detach()) - float(lb.detach())) < 1e-5
    gen = CausalMaskGenerate(8)
    pos = torch.tensor([[0, 1, 2, 0, 1, 0, 1, 2]])
    m = gen(position_ids=pos)[0, 0]
    assert not m[2, 0] and m[3, 2] and m[4, 2] and not m[4, 3] and m[0, 1] and m[7, 4] and not m[7, 5]
    m2 = gen(position_ids=torch.arange(8).unsqueeze(0), actual_seq_len=torch.tensor([[3, 5, 8]]))[0, 0]
    assert torch.equal(m, m2)
    assert CausalMaskGenerate(8, compressed=True)().shape == (2048, 2048)
    sm = FusedScaleMaskSoftmax(scale=0.5)
    p = sm(torch.zeros(1, 1, 8, 8, dtype=torch.bfloat16), m)
    assert p.dtype == torch.bfloat16 and abs(float(p[0, 0, 4].sum()) - 1) < 1e-2 and float(p[0, 0, 4, 2]) == 0.0
    lt = LowerTriangularMask(torch.float32)
    assert lt(True).shape == (128, 128) and lt(False).shape == (1, 1)


def test_weights_loader_streams_an_hf_directory_layer_by_layer(tmp_path):
    """Sharded Hugging Face style directory → lazy index, row / column slices, and a layer-by-layer load that ends in
    the same model (dense Llama and an MoE + MLA model)."""
    from mindformers_b200.checkpoint.io import save_pretrained_dir
    from mindformers_b200.inference.weights_utils import (WeightsLoader, infer_trans_rope_weight, load_weights,
                                                          split_by_tp_rank_columns)
    torch.manual_seed(5)
    ids = torch.randint(0, 1024, (2, 17))
    moe_cfg = dict(num_layers=3, num_moe_experts=4, moe_router_topk=2, moe_ffn_hidden_size=64, first_k_dense_replace=1,
                   moe_shared_expert_intermediate_size=64)
    gated = dict(moe_cfg, use_shared_expert_gating=True)            # Qwen2-MoE: sigmoid gate on the shared expert
    for name, family, kw in (("llama", "llama", {}), ("moe", "qwen3_moe", moe_cfg), ("gated", "qwen2_moe", gated)):
        src = GPTModel(tiny_llama_config(**kw)).eval()
        d = tmp_path / name
        save_pretrained_dir(src, str(d), config_dict={"model_type": family}, max_shard_bytes=400_000, hf_names=True,
                            family=family)
        loader = WeightsLoader(str(d))
        assert len(loader.files) > 2 and loader.has("model.embed_tokens.weight")
        layers, other = loader.layer_groups()
        assert sorted(layers) == list(range(src.config.num_layers)) and "model.norm.weight" in other
        emb = loader.get("model.embed_tokens.weight")
        assert torch.equal(loader.rows("model.embed_tokens.weight", 1, 4), emb[256:512])
        assert torch.equal(split_by_tp_rank_columns(loader.get_slice("model.embed_tokens.weight"), 1, 2), emb[:, 128:])
        dst = GPTModel(tiny_llama_config(**kw)).eval()
        stats = load_weights(dst, str(d), family=family)
        assert stats["layers"] == src.config.num_layers and not stats["missing"]
        total = sum(p.numel() * 4 for p in src.parameters())
        assert stats["peak_group_bytes"] < 0.7 * total              # never the whole model at once
        with torch.no_grad():
            assert torch.equal(src(ids), dst(ids))
    w = torch.arange(12.0).reshape(6, 2)
    assert infer_trans_rope_weight(w, 4)[:, 0].tolist() == [0.0, 2.0, 4.0, 8.0, 6.0, 10.0]


def test_infer_model_mixin_names_strategy_and_name_map(tmp_path):
    import json
    from safetensors.torch import save_file
    from mindformers_b200.inference.model_utils import (convert_net_name, generate_state_dict, save_strategy_file)
    from mindformers_b200.models import AutoModel
    assert convert_net_name("decoder.layers.0.self_attention.linear_k.weight") == \
        "decoder.layers.0.self_attention.linear_qkv.weight"
    assert convert_net_name("decoder.layers.3.mlp.experts.7.gating.weight") == "decoder.layers.3.mlp.experts.weight1"
    assert convert_net_name("decoder.layers.3.mlp.router.weight.weight") == "decoder.layers.3.mlp.router.weight"
    assert convert_net_name("decoder.final_layernorm.weight") == "decoder.final_layernorm.weight"
    cfg = dict(model_type="llama", num_hidden_layers=1, hidden_size=64, num_attention_heads=2, num_key_value_heads=2,
               intermediate_size=128, vocab_size=128, max_position_embeddings=64, params_dtype="float32")
    model = AutoModel.from_config(cfg, device="cpu")
    model.set_phase(False)
    assert not model.is_prefill and model.convert_net_name("a.mlp.gating.weight") == "a.mlp.linear_fc1.weight"
    state = generate_state_dict(model)
    assert state["total_rank"] == 1 and state["model"]["decoder.final_layernorm.weight"]["shard"] == [1]
    path = save_strategy_file(state, str(tmp_path / "strategy" / "ckpt_strategy_rank_0.json"))
    assert json.load(open(path))["model"].keys() == state["model"].keys()
    # a directory with foreign names + param_name_map.json
    new_norm = torch.full((64,), 3.0)
    save_file({"final.norm": new_norm}, str(tmp_path / "w.safetensors"))
    json.dump({"final.norm": "decoder.final_layernorm.weight"}, open(tmp_path / "param_name_map.json", "w"))
    res = model.load_weights_from_dir(str(tmp_path))
    assert res["tensors"] == 1 and torch.equal(dict(model.named_parameters())["decoder.final_layernorm.weight"], new_norm)


def test_micro_batch_interleaved_wrapper():
    from mindformers_b200.wrapper import MicroBatchInterleaved
    torch.manual_seed(2)
    model = GPTModel(tiny_llama_config())
    ids = torch.randint(0, 1024, (4, 17))
    inp, lab = ids[:, :-1].contiguous(), ids[:, 1:].contiguous()
    whole = model(inp, labels=lab)
    wrapped = MicroBatchInterleaved(model, 2)
    split = wrapped(inp, labels=lab)
    assert abs(float(whole.detach()) - float(split.detach())) < 1e-5       # equal token counts per half
    split.backward()
    assert model.output_layer.weight.grad is not None
    with torch.no_grad():
        assert wrapped(inp).shape == model(inp).shape                       # logits are concatenated again
    with pytest.raises(ValueError):
        MicroBatchInterleaved(model, 3)(inp, labels=lab)


def _tiny_train_losses(extra, steps=3):
    import torch
    from mindformers_b200.trainer.engine import TrainingEngine
    torch.manual_seed(0)
    cfg = dict(model_type="llama", vocab_size=128, hidden_size=64, intermediate_size=128, num_hidden_layers=3,
               num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=32)
    eng = TrainingEngine.from_model_config(cfg, device="cpu", dtype="float32", seq_length=32, learning_rate=1e-2, **extra)
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, 128, (2, 33), generator=g)
    batch = {"input_ids": ids[:, :-1], "labels": ids[:, 1:]}
    return eng, [float(eng.train_step(batch)) for _ in range(steps)]


def test_selective_and_full_recompute_and_offload_do_not_change_the_training_curve():
    """Full recompute, selective recompute (default patterns, a pattern that sends a projection back to the recomputed
    set, per-stage counts) and the saved-tensor offload hooks must give the losses of plain training; selective
    recompute must run every matrix product and attention once only per step."""
    from mindformers_b200.ops import functional as Fn
    _, ref = _tiny_train_losses({})
    for extra in (dict(recompute=True), dict(select_recompute=True), dict(select_recompute=[2]),
                  dict(select_recompute=[r"mlp\.linear_fc1", r"mlp\.mul"]),
                  dict(cpu_offloading=True, cpu_offloading_num_layers=2)):
        eng, got = _tiny_train_losses(extra)
        assert all(abs(a - b) < 1e-5 for a, b in zip(ref, got)), (extra, ref, got)
    # inside selective regions every cached operation is computed once and replayed once; a pattern that names a
    # projection takes it out of the cache
    from mindformers_b200.parallel import recompute as R
    seen = {}
    for name, extra in (("selective", dict(select_recompute=True)), ("selective_fc1", dict(select_recompute=[r"mlp\.linear_fc1"]))):
        R.STATS.update(computed=0, replayed=0)
        _tiny_train_losses(extra, steps=1)
        seen[name] = dict(R.STATS)
    assert seen["selective"]["computed"] == seen["selective"]["replayed"] > 0, seen
    assert 0 < seen["selective_fc1"]["replayed"] < seen["selective"]["replayed"], seen


def test_packed_rows_attend_inside_their_documents_only():
    """``actual_seq_len`` (cumulative document ends per row, what the GPT dataset emits with the compressed EOD mask)
    reaches the attention layers: the logits of the second document of a packed row equal those of the same tokens fed
    alone, with position ids reset at the boundary."""
    import torch
    from mindformers_b200.parallel.layers.gpt_model import GPTModel
    from mindformers_b200.parallel.transformer_config import TransformerConfig
    torch.manual_seed(0)
    cfg = TransformerConfig(num_layers=2, hidden_size=64, num_attention_heads=4, num_query_groups=2, ffn_hidden_size=128,
                            vocab_size=97, seq_length=16, max_position_embeddings=16, params_dtype="float32",
                            compute_dtype="float32")
    cfg.device = "cpu"
    model = GPTModel(cfg).eval()
    ids = torch.randint(1, 97, (2, 16))
    cut = [6, 11]                                        # row 0: documents [0,6) and [6,16); row 1: [0,11), [11,16)
    asl = torch.tensor([[6, 16, 16, 16], [11, 16, 16, 16]], dtype=torch.int32)
    pos = torch.stack([torch.cat([torch.arange(c), torch.arange(16 - c)]) for c in cut])
    with torch.no_grad():
        packed = model(ids, position_ids=pos, actual_seq_len=asl).view(2, 16, -1)
        plain = model(ids, position_ids=pos).view(2, 16, -1)
        for b, c in enumerate(cut):
            alone = model(ids[b:b + 1, c:], position_ids=torch.arange(16 - c).unsqueeze(0)).view(16 - c, -1)
            assert torch.allclose(packed[b, c:], alone, atol=1e-5)
            assert not torch.allclose(plain[b, c:], alone, atol=1e-3)      # without the table the documents leak
            assert torch.allclose(packed[b, :c], plain[b, :c], atol=1e-5)  # the first document never sees the second


def _tiny_mla_config(**kw):
    base = dict(num_layers=2, hidden_size=128, num_attention_heads=4, ffn_hidden_size=256, vocab_size=512,
                seq_length=64, max_position_embeddings=64, params_dtype="float32", compute_dtype="float32",
                q_lora_rank=32, kv_lora_rank=32, qk_head_dim=32, qk_pos_emb_head_dim=16, v_head_dim=32,
                rotary_scaling_factor=1.0)
    base.update(kw)
    cfg = MLATransformerConfig(**base)
    cfg.device = "cpu"
    return cfg


@pytest.mark.parametrize("q_rank", [32, None])
def test_mla_with_one_module_per_projection_matches_the_concatenated_layout(q_rank):
    """``mla_qkv_concat=False`` builds ``linear_q_down_proj / linear_q_up_proj / linear_kv_down_proj /
    linear_kv_up_proj / kv_layernorm`` (``linear_q_proj`` without query compression). A state dict of the
    concatenated model, split into per-projection names and loaded into that model, gives the same logits and
    gradients."""
    from mindformers_b200.checkpoint.name_maps import fuse_state_dict, unfuse_state_dict
    from mindformers_b200.parallel.layers.attention import MLASelfAttentionMegatron
    torch.manual_seed(21)
    a = GPTModel(_tiny_mla_config(q_lora_rank=q_rank))
    b = GPTModel(_tiny_mla_config(q_lora_rank=q_rank, mla_qkv_concat=False))
    attn = b.decoder.layers[0].self_attention
    assert isinstance(attn, MLASelfAttentionMegatron)
    names = {n for n, _ in b.named_parameters()}
    want = ["linear_kv_down_proj.weight", "linear_kv_up_proj.weight", "kv_layernorm.weight", "linear_proj.weight"]
    want += ["linear_q_down_proj.weight", "linear_q_up_proj.weight", "q_layernorm.weight"] if q_rank else ["linear_q_proj.weight"]
    for w in want:
        assert f"decoder.layers.0.self_attention.{w}" in names, w
    assert not any("linear_qkv" in n or "linear_kvb" in n or ".k_layernorm" in n for n in names)
    per_proj = unfuse_state_dict(a.state_dict(), a.config)
    fused_for_b = fuse_state_dict(per_proj, b.config)
    missing, unexpected = b.load_state_dict(fused_for_b, strict=False)
    assert not [m for m in missing if "rotary" not in m] and not unexpected, (missing, unexpected)
    ids = torch.randint(0, 512, (2, 33))
    la = a(ids[:, :-1].contiguous(), ids[:, 1:].contiguous())
    lb = b(ids[:, :-1].contiguous(), ids[:, 1:].contiguous())
    assert torch.allclose(la, lb, atol=1e-5)
    la.backward(), lb.backward()
    ga = a.decoder.layers[1].self_attention.linear_kvb.weight.grad
    gb = b.decoder.layers[1].self_attention.linear_kv_up_proj.weight.grad
    assert torch.allclose(ga, gb, atol=1e-5)
    # and back: the per-projection model's own state dict fuses into the concatenated layout
    back = fuse_state_dict(b.state_dict(), a.config)
    assert set(back) == set(a.state_dict())


def test_cross_attention_matches_an_fp32_reference():
    """Queries from the decoder states, keys / values from an encoder sequence of another length; no mask."""
    from mindformers_b200.parallel.layers.attention import AttnMeta, CrossAttention
    torch.manual_seed(22)
    cfg = tiny_llama_config(hidden_size=64, num_attention_heads=4, num_query_groups=4, add_qkv_bias=True)
    ca = CrossAttention(cfg)
    names = {n for n, _ in ca.named_parameters()}
    assert {"linear_q.weight", "linear_kv.weight", "linear_proj.weight", "linear_q.bias", "linear_kv.bias"} <= names
    assert ca.linear_kv.weight.shape == (128, 64)
    B, Sq, Sk, H, nh, hd = 2, 5, 9, 64, 4, 16
    x = torch.randn(B * Sq, H, requires_grad=True)
    mem = torch.randn(B * Sk, H)
    out, _ = ca(x, mem, AttnMeta(batch=B, seq_len=Sq))
    q = (x @ ca.linear_q.weight.t() + ca.linear_q.bias).view(B, Sq, nh, hd).transpose(1, 2)
    kv = mem @ ca.linear_kv.weight.t() + ca.linear_kv.bias
    k = kv[:, :H].reshape(B, Sk, nh, hd).transpose(1, 2)
    v = kv[:, H:].reshape(B, Sk, nh, hd).transpose(1, 2)
    p = torch.softmax(q @ k.transpose(-1, -2) / hd ** 0.5, dim=-1)
    ref = (p @ v).transpose(1, 2).reshape(B * Sq, H) @ ca.linear_proj.weight.t()
    assert torch.allclose(out, ref, atol=1e-5)
    out.sum().backward()
    assert x.grad is not None and ca.linear_kv.weight.grad.abs().sum() > 0
    with pytest.raises(ValueError):
        CrossAttention(tiny_llama_config(hidden_size=64, num_attention_heads=4, num_query_groups=2))


def test_legacy_llama_emits_and_takes_the_legacy_parameter_names(tmp_path):
    """Built from legacy keys (``num_heads``, ``n_kv_heads``, ``multiple_of``), it lists its weights as
    ``model.layers.N.attention.wq`` … (views of the fused tensors), loads such a dict (also through the checkpoint
    reader, and in the ``qkv_concat`` spelling) and then computes what the source model computes."""
    from safetensors.torch import save_file
    from mindformers_b200.checkpoint.io import load_checkpoint
    from mindformers_b200.models import LegacyLlamaForCausalLM, LlamaLegacyConfig
    from mindformers_b200.models.llama_legacy import legacy_ffn_hidden_size
    assert legacy_ffn_hidden_size(4096, None, 256, None) == 11008           # Llama-2 7B
    assert legacy_ffn_hidden_size(4096, None, 1024, 1.3) == 14336           # Llama-3 8B
    torch.manual_seed(23)
    kw = dict(num_layers=2, num_heads=4, n_kv_heads=2, hidden_size=64, multiple_of=32, vocab_size=256, seq_length=32,
              params_dtype="float32")
    src = LegacyLlamaForCausalLM(LlamaLegacyConfig(**kw), device="cpu").eval()
    assert src.config.ffn_hidden_size == 192 and src.config.num_query_groups == 2
    sd = src.state_dict()
    for k in ("model.tok_embeddings.embedding_weight", "model.layers.1.attention.wq.weight",
              "model.layers.1.attention.wk.weight", "model.layers.0.attention.wo.weight",
              "model.layers.0.feed_forward.w1.weight", "model.layers.0.feed_forward.w2.weight",
              "model.layers.0.feed_forward.w3.weight", "model.layers.0.attention_norm.weight",
              "model.layers.0.ffn_norm.weight", "model.norm_out.weight", "lm_head.weight"):
        assert k in sd, (k, sorted(sd)[:12])
    assert sd["model.layers.1.attention.wk.weight"].shape == (32, 64)
    fused = src.model.decoder.layers[1].self_attention.linear_qkv.weight
    assert sd["model.layers.1.attention.wq.weight"].data_ptr() == fused.data_ptr()          # a view, not a copy
    ids = torch.randint(0, 256, (2, 16))
    with torch.no_grad():
        want = src(ids)
    dst = LegacyLlamaForCausalLM(LlamaLegacyConfig(**kw), device="cpu").eval()
    dst.load_state_dict({k: v.clone() for k, v in sd.items()})
    with torch.no_grad():
        assert torch.equal(dst(ids), want)
    # the fused legacy spelling (qkv_concat) and the generic checkpoint reader
    cat = LegacyLlamaForCausalLM(LlamaLegacyConfig(qkv_concat=True, **kw), device="cpu").eval()
    cat.load_state_dict({k: v.clone() for k, v in sd.items()})
    sd_cat = cat.state_dict()
    assert "model.layers.0.attention.w_qkv.weight" in sd_cat and "model.layers.0.feed_forward.w_gate_hidden.weight" in sd_cat
    assert not any(".attention.wq." in k for k in sd_cat)
    save_file({k: v.contiguous() for k, v in sd_cat.items()}, str(tmp_path / "legacy.safetensors"))
    plain = GPTModel(tiny_llama_config(num_layers=2, num_attention_heads=4, num_query_groups=2, hidden_size=64,
                                       ffn_hidden_size=192, vocab_size=256, seq_length=32)).eval()
    load_checkpoint(plain, str(tmp_path / "legacy.safetensors"), strict=True)
    with torch.no_grad():
        assert torch.allclose(plain(ids), want, atol=1e-6)


def _chatglm_reference_forward(sd, ids, nh, nkv, hd, eps, base):
    """ChatGLM / GLM-4 forward written from the published architecture: fused query_key_value with bias, rotary on the
    first half of each head over adjacent pairs, grouped KV heads, RMSNorm, SwiGLU from one fused projection."""
    B, S = ids.shape
    x = sd["transformer.embedding.word_embeddings.weight"][ids]
    rot = hd // 2
    theta = 1.0 / (base ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))
    ang = torch.outer(torch.arange(S, dtype=torch.float32), theta)              # [S, rot/2]
    cos, sin = ang.cos()[None, :, None, :], ang.sin()[None, :, None, :]

    def rope(t):                                                                # t [B, S, h, hd]
        r, p = t[..., :rot], t[..., rot:]
        r = r.reshape(*r.shape[:-1], rot // 2, 2)
        a, b = r[..., 0], r[..., 1]
        out = torch.stack((a * cos - b * sin, b * cos + a * sin), dim=-1).flatten(-2)
        return torch.cat((out, p), dim=-1)

    def rms(t, w):
        return t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + eps) * w

    n_layers = 1 + max(int(k.split(".")[3]) for k in sd if k.startswith("transformer.encoder.layers."))
    for i in range(n_layers):
        pre = f"transformer.encoder.layers.{i}."
        h = rms(x, sd[pre + "input_layernorm.weight"])
        qkv = h @ sd[pre + "self_attention.query_key_value.weight"].t() + sd[pre + "self_attention.query_key_value.bias"]
        q, k, v = qkv.split([nh * hd, nkv * hd, nkv * hd], dim=-1)
        q, k, v = q.view(B, S, nh, hd), k.view(B, S, nkv, hd), v.view(B, S, nkv, hd)
        q, k = rope(q), rope(k)
        k, v = (t.repeat_interleave(nh // nkv, dim=2) for t in (k, v))
        s = torch.einsum("bqhd,bkhd->bhqk", q, k) / hd ** 0.5
        s = s.masked_fill(torch.ones(S, S, dtype=torch.bool).triu(1), float("-inf"))
        o = torch.einsum("bhqk,bkhd->bqhd", s.softmax(-1), v).reshape(B, S, nh * hd)
        x = x + o @ sd[pre + "self_attention.dense.weight"].t()
        h = rms(x, sd[pre + "post_attention_layernorm.weight"])
        gate, up = (h @ sd[pre + "mlp.dense_h_to_4h.weight"].t()).chunk(2, dim=-1)
        x = x + (torch.nn.functional.silu(gate) * up) @ sd[pre + "mlp.dense_4h_to_h.weight"].t()
    x = rms(x, sd["transformer.encoder.final_layernorm.weight"])
    return x @ sd["transformer.output_layer.weight"].t()


def test_glm4_checkpoint_loads_and_reproduces_the_published_architecture(tmp_path):
    """A checkpoint with GLM-4's own key names and tensor layouts, written as a pretrained directory, loads into
    ``ChatGLM2ForConditionalGeneration``; the logits equal an independent forward of the GLM architecture (partial,
    pair-wise rotary embedding, QKV bias, 2 KV groups), and saving with the family's names gives the tensors back."""
    import json
    from safetensors.torch import save_file
    from mindformers_b200.checkpoint import name_maps
    from mindformers_b200.models import ChatGLM2Config, ChatGLM2ForConditionalGeneration
    torch.manual_seed(24)
    H, F, nh, nkv, hd, V, L = 64, 96, 4, 2, 16, 128, 2
    sd = {"transformer.embedding.word_embeddings.weight": torch.randn(V, H) * 0.1,
          "transformer.encoder.final_layernorm.weight": 1 + 0.1 * torch.randn(H),
          "transformer.output_layer.weight": torch.randn(V, H) * 0.1,
          "transformer.rotary_pos_emb.inv_freq": torch.zeros(hd // 4)}
    for i in range(L):
        pre = f"transformer.encoder.layers.{i}."
        sd[pre + "input_layernorm.weight"] = 1 + 0.1 * torch.randn(H)
        sd[pre + "post_attention_layernorm.weight"] = 1 + 0.1 * torch.randn(H)
        sd[pre + "self_attention.query_key_value.weight"] = torch.randn((nh + 2 * nkv) * hd, H) * 0.1
        sd[pre + "self_attention.query_key_value.bias"] = torch.randn((nh + 2 * nkv) * hd) * 0.1
        sd[pre + "self_attention.dense.weight"] = torch.randn(H, nh * hd) * 0.1
        sd[pre + "mlp.dense_h_to_4h.weight"] = torch.randn(2 * F, H) * 0.1
        sd[pre + "mlp.dense_4h_to_h.weight"] = torch.randn(H, F) * 0.1
    cfg_json = dict(model_type="chatglm", num_layers=L, padded_vocab_size=V, hidden_size=H, ffn_hidden_size=F,
                    kv_channels=hd, num_attention_heads=nh, multi_query_attention=True, multi_query_group_num=nkv,
                    seq_length=32, layernorm_epsilon=1e-5, rope_ratio=50.0, rmsnorm=True, add_qkv_bias=True,
                    add_bias_linear=False, torch_dtype="float32", post_layer_norm=True,
                    apply_query_key_layer_scaling=True)
    d = tmp_path / "glm4"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(cfg_json))
    save_file(sd, str(d / "model.safetensors"))
    model = ChatGLM2ForConditionalGeneration.from_pretrained(str(d), strict=True, device="cpu").eval()
    c = model.config
    assert (c.num_query_groups, c.rotary_percent, c.rotary_interleaved, c.add_qkv_bias, c.add_bias_linear) == \
        (nkv, 0.5, True, True, False)
    assert c.rotary_base == 500000.0 and c.vocab_size == V and c.normalization == "RMSNorm"
    ids = torch.randint(0, V, (2, 24))
    with torch.no_grad():
        got = model(ids)
    ref = _chatglm_reference_forward(sd, ids, nh, nkv, hd, 1e-5, 500000.0)
    got = got.reshape(ref.shape)
    assert torch.allclose(got, ref, atol=2e-5), (got - ref).abs().max()
    back = name_maps.framework_to_hf(dict(model.named_parameters()), model.config, "glm")
    assert set(back) == set(sd) - {"transformer.rotary_pos_emb.inv_freq"}
    for k, v in back.items():
        assert torch.equal(v, sd[k]), k
    assert ChatGLM2Config().to_transformer_dict()["multi_query_group_num"] == 2


def test_shard_checkpoint_and_pipeline_stage_check():
    from mindformers_b200.models import LlamaConfig, LlamaForCausalLM
    from mindformers_b200.models.modeling_utils import shard_checkpoint
    sd = {f"w{i}": torch.zeros(n, dtype=torch.float32) for i, n in enumerate([1500, 1500, 500, 1500, 500, 500])}
    shards, index = shard_checkpoint(sd, max_shard_size=10000, weights_name="model.safetensors")
    assert [sorted(v) for v in shards.values()] == [["w0"], ["w1", "w2"], ["w3", "w4", "w5"]]     # in key order, no packing
    assert list(shards)[0] == "model-00001-of-00003.safetensors" and index["weight_map"]["w4"] == "model-00003-of-00003.safetensors"
    assert index["metadata"]["total_size"] == 6000 * 4
    one, idx = shard_checkpoint(sd, "1MB")
    assert list(one) == ["model.safetensors"] and idx is None
    big, _ = shard_checkpoint({"a": torch.zeros(10), "huge": torch.zeros(10000), "b": torch.zeros(10)}, 1000)
    assert [sorted(v) for v in big.values()] == [["a"], ["huge"], ["b"]]
    model = LlamaForCausalLM(LlamaConfig(vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=3,
                                         num_attention_heads=2, params_dtype="float32"), device="cpu")
    model.check_pipeline_stage(2)
    model.check_pipeline_stage(1, 8)
    with pytest.raises(ValueError, match="at least pipeline_stage"):
        model.check_pipeline_stage(4)
    with pytest.raises(ValueError, match="pp_interleave_num"):
        model.check_pipeline_stage(2, 2)


def test_hidden_and_attention_dropout_act_in_training_only():
    """``hidden_dropout`` masks the sub-layer outputs before the residual add and ``attention_dropout`` the attention
    probabilities: two training passes differ, evaluation is deterministic and equals the model without dropout."""
    torch.manual_seed(41)
    plain = GPTModel(tiny_llama_config())
    torch.manual_seed(41)
    drop = GPTModel(tiny_llama_config(hidden_dropout=0.2, attention_dropout=0.1))
    drop.load_state_dict(plain.state_dict())
    ids = torch.randint(0, 1024, (2, 33))
    inp, lab = ids[:, :-1].contiguous(), ids[:, 1:].contiguous()
    drop.train()
    a, b = drop(inp, lab), drop(inp, lab)
    assert abs(float(a) - float(b)) > 1e-6
    a.backward()
    assert all(p.grad is not None for p in drop.parameters())
    drop.eval(), plain.eval()
    with torch.no_grad():
        assert torch.equal(drop(inp, lab), plain(inp, lab))
    only_hidden = GPTModel(tiny_llama_config(hidden_dropout=0.5)).train()
    x = only_hidden(inp, lab)
    assert torch.isfinite(x)


def test_build_model_config_and_base_model_alias(tmp_path):
    """YAML-style builders: a configuration by registered class name or by model type, a network from the ``model``
    section, and the older ``BaseModel`` base with ``load_checkpoint`` from ``checkpoint_name_or_path``."""
    from mindformers_b200.models import BaseModel, LlamaConfig, LlamaForCausalLM, build_model, build_model_config
    kw = dict(hidden_size=64, num_hidden_layers=1, num_attention_heads=4, vocab_size=96, intermediate_size=128)
    assert isinstance(build_model_config({"type": "LlamaConfig", **kw}), LlamaConfig)
    assert type(build_model_config({"model_type": "qwen2", **kw})).__name__ == "Qwen2Config"
    assert build_model_config(None) is None
    section = {"arch": {"type": "LlamaForCausalLM"},
               "model_config": {"type": "LlamaConfig", "params_dtype": "float32", "compute_dtype": "float32", **kw}}
    net = build_model(section, default_args={"device": "cpu"})
    assert isinstance(net, LlamaForCausalLM)
    net.save_pretrained(str(tmp_path / "m"))

    class Mine(BaseModel):
        config_class = LlamaConfig
    cfg = LlamaConfig(params_dtype="float32", compute_dtype="float32", checkpoint_name_or_path=str(tmp_path / "m"), **kw)
    other = Mine(cfg, device="cpu")
    other.load_checkpoint(cfg)
    for (n, a), (_, b) in zip(net.state_dict().items(), other.state_dict().items()):
        assert torch.equal(a, b), n


def test_legacy_moe_config_section_builds_the_experts():
    """The older top-level ``moe_config`` section (TeleChat2-39B-A12B style YAML) reaches the model: expert count, top-k,
    router dtype and the load-balancing coefficient; keys that only select the reference's code paths are dropped; a
    dense model that carries the section's defaults stays dense."""
    import os
    import yaml
    from mindformers_b200.models import build_network, merge_moe_config
    from mindformers_b200.trainer.base_trainer import _model_dict
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = yaml.safe_load(open(os.path.join(root, "configs", "telechat2", "finetune_telechat2_39b_a12b.yaml")))
    mc = _model_dict(cfg)
    assert mc["expert_num"] == 16 and mc["num_experts_chosen"] == 4 and mc["router_aux_loss_coef"] == 0.01
    assert "routing_policy" not in mc and "capacity_factor" not in mc and "shared_expert_num" not in mc
    assert merge_moe_config({"hidden_size": 8}, {"expert_num": 1, "num_experts_chosen": 1}) == {"hidden_size": 8}
    assert merge_moe_config({"expert_num": 4}, {"expert_num": 8})["expert_num"] == 4          # the model section wins
    small = dict(mc, num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=4, intermediate_size=96,
                 moe_intermediate_size=48, vocab_size=128, max_position_embeddings=64, seq_length=64, params_dtype="float32",
                 compute_dtype="float32", device="cpu", fused_moe_comm=False)
    net = build_network({"model_config": small})
    tc = net.model.config
    assert tc.num_moe_experts == 16 and tc.moe_router_topk == 4 and abs(tc.moe_aux_loss_coeff - 0.01) < 1e-12
    names = [n for n, _ in net.named_parameters()]
    assert any("experts" in n for n in names) and any("router" in n for n in names)
    ids = torch.randint(0, 128, (2, 16))
    loss = net.model(ids, ids)
    loss = loss[0] if isinstance(loss, tuple) else loss
    loss.float().mean().backward()
    # the section nested under model_config works as well
    nested = build_network({"model_config": dict({k: v for k, v in small.items() if k not in ("expert_num", "num_experts_chosen",
                                                                                               "router_aux_loss_coef",
                                                                                               "router_dense_type",
                                                                                               "balance_via_topk_bias",
                                                                                               "topk_bias_update_rate")},
                                                 moe_config={"expert_num": 8, "num_experts_chosen": 2})})
    assert nested.model.config.num_moe_experts == 8 and nested.model.config.moe_router_topk == 2
