"""Legacy building blocks, quantisers, loss scale, RNG tracker, sequence-pipeline split (CPU)."""
import math

import torch

from mindformers_b200.core.loss_scale import AdaptiveLossScaleUpdateCell, DynamicLossScaleUpdateCell
from mindformers_b200.modules import (AlibiTensor, FreqsMgr, LayerNorm, Linear, MoEConfig, MoEV2, SequenceSplit,
                                      get_activation, get_rng_tracker, model_parallel_manual_seed)
from mindformers_b200.modules import quantizers as Q


def test_freqs_mgr_extension_methods():
    base = FreqsMgr(64, 128, 128, theta=10000.0)
    cos, sin = base()
    assert cos.shape == (128, 64) and torch.allclose(cos[0], torch.ones(64))
    pi = FreqsMgr(64, 128, 128, scaling_factor=4.0, extend_method="PI")
    assert torch.allclose(pi.freqs_cos[4], base.freqs_cos[1], atol=1e-6)        # positions shrink by the factor
    ntk = FreqsMgr(64, 128, 128, scaling_factor=4.0, extend_method="NTK")
    assert ntk.freqs_sin[1, 31] < base.freqs_sin[1, 31]                          # lowest frequency slowed down
    l3 = FreqsMgr(128, 64, 64, theta=500000.0, scaling_factor=8.0, extend_method="LLAMA3", original_max_position=8192)
    plain = FreqsMgr(128, 64, 64, theta=500000.0)
    assert torch.allclose(l3.freqs_cos[:, 0], plain.freqs_cos[:, 0])             # high frequencies untouched
    assert not torch.allclose(l3.freqs_sin[:, 63], plain.freqs_sin[:, 63])
    yarn = FreqsMgr(64, 64, 64, scaling_factor=4.0, extend_method="YARN", original_max_position=32)
    assert yarn.mscale > 1.0


def test_linear_layernorm_alibi_activation():
    torch.manual_seed(0)
    lin = Linear(16, 8, activation="gelu", compute_dtype=torch.float32)
    x = torch.randn(4, 16)
    want = torch.nn.functional.gelu(x @ lin.weight.t() + lin.bias, approximate="tanh")
    assert torch.allclose(lin(x), want, atol=1e-5)
    ex = Linear(16, 8, expert_num=3, compute_dtype=torch.float32)
    assert ex(torch.randn(3, 5, 16)).shape == (3, 5, 8)
    ln = LayerNorm(16)
    assert torch.allclose(ln(x).mean(-1), torch.zeros(4), atol=1e-5)
    bias = AlibiTensor(8, 4)(torch.ones(2, 8))
    assert bias.shape == (2, 4, 1, 8) and bias[0, 0, 0, 7] > bias[0, 0, 0, 0]
    assert get_activation("swiglu")(torch.randn(3, 8)).shape == (3, 4)


def test_capacity_moe_drops_and_aux():
    torch.manual_seed(1)
    cfg = MoEConfig(expert_num=4, capacity_factor=0.5, num_experts_chosen=2, moe_intermediate_size=16, aux_loss_types=["expert", "device"],
                    aux_loss_factors=[0.01, 0.01], devices_per_group=2, shared_expert_num=1)
    moe = MoEV2(32, 64, cfg)
    x = torch.randn(2, 16, 32, requires_grad=True)
    y, aux = moe(x)
    assert y.shape == x.shape and aux.item() > 0
    assert 0.0 < float(moe.router.last_drop_rate) < 1.0          # capacity 0.5 must drop something
    (y.sum() + aux).backward()
    assert moe.w1.grad is not None and x.grad is not None
    cfg2 = MoEConfig(expert_num=4, capacity_factor=8.0, num_experts_chosen=2, moe_intermediate_size=16, enable_sdrop=True)
    moe2 = MoEV2(32, 64, cfg2)
    moe2(x)
    assert float(moe2.router.last_drop_rate) == 0.0


def test_quantizers_roundtrip_and_model():
    torch.manual_seed(2)
    w = torch.randn(64, 128)
    for dt, tol in (("int8", 0.01), ("int4", 0.15)):
        q, s = Q.quantize_weight_rtn(w, dt, group_size=32)
        assert ((Q.dequantize_weight(q, s, torch.float32) - w).norm() / w.norm()) < tol
    kq, ks = Q.quantize_kv_int8(torch.randn(4, 2, 64))
    assert kq.dtype == torch.int8 and ks.shape == (4, 2, 1)
    from mindformers_b200.models import LlamaConfig, LlamaForCausalLM
    cfg = LlamaConfig(vocab_size=64, hidden_size=128, intermediate_size=256, num_hidden_layers=1, num_attention_heads=4,
                      num_key_value_heads=2, params_dtype="float32", compute_dtype="float32")
    m = LlamaForCausalLM(cfg, device="cpu").eval()
    ids = torch.randint(0, 64, (1, 16))
    ref = m(ids)
    stats = Q.collect_activation_absmax(m, [ids], lambda mod, b: mod(b))
    n = Q.quantize_model(m, Q.SmoothQuantConfig(), stats)
    assert n == 4
    got = m(ids)
    assert (got - ref).norm() / ref.norm() < 0.08
    m2 = LlamaForCausalLM(cfg, device="cpu").eval()
    ref2 = m2(ids)
    assert Q.quantize_model(m2, Q.Fp8BlockConfig()) == 4
    assert (m2(ids) - ref2).norm() / ref2.norm() < 0.1


def test_loss_scale_rng_and_sequence_split():
    ls = DynamicLossScaleUpdateCell(1024, 2, 3)
    assert ls.update(True) == 512 and [ls.update(False) for _ in range(3)][-1] == 1024
    ad = AdaptiveLossScaleUpdateCell(1024, 2, 100, max_scale_window=100, min_scale_window=25)
    ad.update(True)
    assert ad.window == 50
    model_parallel_manual_seed(5)
    tr = get_rng_tracker()
    with tr.fork():
        a = torch.rand(3)
    with tr.fork():
        b = torch.rand(3)
    assert not torch.equal(a, b)
    model_parallel_manual_seed(5)
    with get_rng_tracker().fork():
        assert torch.equal(torch.rand(3), a)
    parts = SequenceSplit(4).split({"input_ids": torch.arange(32).view(2, 16), "labels": torch.arange(32).view(2, 16)})
    assert len(parts) == 4 and parts[2]["input_ids"].shape == (2, 4) and parts[2]["position_ids"][0, 0] == 8


def test_apply_fn_runs_forward_directly_without_gradients():
    """With gradients off an autograd Function's forward runs as a plain call on a throw-away context; with gradients
    on it goes through ``Function.apply`` and differentiates as usual."""
    import torch
    from mindformers_b200.ops.functional import apply_fn

    class Scale(torch.autograd.Function):
        calls = []

        @staticmethod
        def forward(ctx, x, k):
            Scale.calls.append(type(ctx).__name__)
            ctx.save_for_backward(x)
            ctx.k = k
            ctx.mark_non_differentiable()
            return x * k

        @staticmethod
        def backward(ctx, g):
            return g * ctx.k, None

    x = torch.arange(4.0, requires_grad=True)
    y = apply_fn(Scale, x, 3.0)
    y.sum().backward()
    assert torch.equal(x.grad, torch.full((4,), 3.0))
    with torch.no_grad():
        z = apply_fn(Scale, x, 3.0)
    assert torch.equal(z, y.detach()) and not z.requires_grad
    assert Scale.calls[0] != "_NoGradCtx" and Scale.calls[1] == "_NoGradCtx"


def test_init_methods():
    import torch
    from mindformers_b200.parallel.init_method import init_method_normal, init_method_zero, scaled_init_method_normal
    torch.manual_seed(0)
    a = init_method_normal(0.02)(torch.empty(512, 512))
    b = scaled_init_method_normal(0.02, 8)(torch.empty(512, 512))
    assert abs(a.std().item() - 0.02) < 1e-3 and abs(b.std().item() - 0.02 / 4.0) < 3e-4
    assert init_method_zero()(torch.ones(3)).abs().sum() == 0


def test_batched_expert_linears_match_a_per_expert_loop():
    import torch
    from mindformers_b200.parallel.layers.tensor_parallel import ColumnParallelBatchedLinear, RowParallelBatchedLinear
    from mindformers_b200.parallel.transformer_config import TransformerConfig
    cfg = TransformerConfig(num_layers=1, hidden_size=32, num_attention_heads=2, ffn_hidden_size=64, vocab_size=64,
                            num_moe_experts=4, moe_router_topk=2, moe_ffn_hidden_size=48, params_dtype="float32",
                            compute_dtype="float32")
    cfg.device = "cpu"
    torch.manual_seed(0)
    up = ColumnParallelBatchedLinear(32, 48, config=cfg)
    down = RowParallelBatchedLinear(48, 32, config=cfg)
    assert up.weight.shape == (4, 48, 32) and down.weight.shape == (4, 32, 48) and up.weight.is_expert
    x = torch.randn(4, 5, 32, requires_grad=True)
    h, _ = up(x)
    y, _ = down(torch.nn.functional.silu(h))
    ref = torch.stack([torch.nn.functional.silu(x[e] @ up.weight[e].t()) @ down.weight[e].t() for e in range(4)])
    assert torch.allclose(y, ref, atol=1e-5)
    y.sum().backward()
    assert x.grad is not None and up.weight.grad.shape == up.weight.shape
    import pytest
    with pytest.raises(ValueError):
        ColumnParallelBatchedLinear(32, 48, config=cfg, is_expert=False)


def test_local_block_sparse_attention_matches_dense_masked_attention():
    import torch
    from mindformers_b200.modules.local_block_sparse_attention import LocalBlockSparseAttention
    torch.manual_seed(0)
    att = LocalBlockSparseAttention(seq_len=64, size_per_head=16, local_size=32, block_size=8, dropout_rate=0.0).eval()
    q, k, v = (torch.randn(2, 3, 64, 16) for _ in range(3))
    out = att(q, k, v)
    mask = att.dense_mask()
    assert mask[40, 40] and mask[40, 16] and not mask[40, 15] and not mask[40, 41]      # window of 4 blocks, causal
    s = (q @ k.transpose(-1, -2)) / 4.0
    ref = torch.softmax(s.masked_fill(~mask, float("-inf")), -1) @ v
    assert torch.allclose(out, ref, atol=1e-5)
    pad = torch.ones(2, 64, 64)
    pad[1, :, :5] = 0                                   # batch 1 may not look at its first five tokens
    out2 = att(q, k, v, pad)
    ref2 = torch.softmax(s.masked_fill(~(mask & pad.bool()[:, None]), float("-inf")), -1)
    ref2 = torch.nan_to_num(ref2, nan=0.0) @ v
    assert torch.allclose(out2, ref2, atol=1e-5) and torch.allclose(out2[0], out[0], atol=1e-6)


def test_moe_infer_matches_per_token_loop():
    import torch
    from mindformers_b200.modules import MoEConfig, MoEInfer
    cfg = MoEConfig(expert_num=4, num_experts_chosen=2, moe_intermediate_size=12)
    torch.manual_seed(1)
    moe = MoEInfer(8, 12, cfg)
    x = torch.randn(2, 5, 8)
    out = moe(x)
    assert out.shape == x.shape and not out.requires_grad
    probs, ids, _ = moe.route(x.reshape(-1, 8))
    ref = torch.zeros(10, 8)
    for t in range(10):
        for j in range(2):
            e = int(ids[t, j])
            g, u = (x.reshape(-1, 8)[t] @ moe.w1[e]).chunk(2)
            ref[t] += probs[t, j] * ((torch.nn.functional.silu(g) * u) @ moe.w2[e])
    assert torch.allclose(out.reshape(-1, 8), ref.detach(), atol=1e-5)


def test_infer_attention_paged_and_contiguous_caches_match_full_attention():
    """Prefill + two decode steps through the paged cache manager and through the contiguous cache manager give the
    attention of the whole sequence recomputed from scratch (with RoPE)."""
    import torch
    from mindformers_b200.inference.block_manager import BlockTables
    from mindformers_b200.modules import InferAttention
    from mindformers_b200.ops import functional as Fn
    torch.manual_seed(0)
    nh, nkv, hd, B, S0, steps = 4, 2, 16, 2, 5, 2
    total = S0 + steps
    q_all, k_all, v_all = (torch.randn(B, total, n * hd) for n in (nh, nkv, nkv))
    inv = 1.0 / (10000 ** (torch.arange(0, hd, 2).float() / hd))
    ang = torch.arange(64).float()[:, None] * inv[None]
    freqs = (ang.cos(), ang.sin())

    def reference(upto):
        pos = torch.arange(upto).repeat(B)
        q = Fn.rope_reference(q_all[:, :upto].reshape(B * upto, nh, hd), *freqs, pos, nh, hd).view(B, upto, nh, hd)
        k = Fn.rope_reference(k_all[:, :upto].reshape(B * upto, nkv, hd), *freqs, pos, nkv, hd).view(B, upto, nkv, hd)
        v = v_all[:, :upto].view(B, upto, nkv, hd)
        return Fn.attention_reference(q, k, v, causal=True).reshape(B, upto, nh * hd)

    paged = InferAttention(nh, hd, nkv, block_size=4, num_blocks=16, compute_dtype=torch.float32, device="cpu")
    dense = InferAttention(nh, hd, nkv, use_paged_attention=False, max_batch_size=B, max_seq_length=16,
                           compute_dtype=torch.float32, device="cpu")
    tables = BlockTables(16, 4, 16)
    tables.init_cache_engine(B)
    table, slots = tables.assemble_pa_full_inputs([S0] * B)
    pos = torch.arange(S0).repeat(B)
    flat = lambda t, a, b: t[:, a:b].reshape(B * (b - a), -1)
    out = paged(flat(q_all, 0, S0), flat(k_all, 0, S0), flat(v_all, 0, S0), tables.context_lens(), table, slots, freqs,
                pos, [S0] * B, True)
    ref = reference(S0)
    assert torch.allclose(out.view(B, S0, -1), ref, atol=1e-5)
    out_d = dense(q_all[:, :S0], k_all[:, :S0], v_all[:, :S0], torch.tensor([S0] * B), freqs_cis=freqs, is_prefill=True)
    assert torch.allclose(out_d, ref, atol=1e-5)
    for step in range(steps):
        t = S0 + step
        table, slots = tables.assemble_pa_inc_inputs(None, 1)
        pos = torch.full((B,), t)
        out = paged(flat(q_all, t, t + 1), flat(k_all, t, t + 1), flat(v_all, t, t + 1), tables.context_lens(), table,
                    slots, freqs, pos, None, False)
        ref = reference(t + 1)[:, -1]
        assert torch.allclose(out, ref, atol=1e-5), step
        out_d = dense(q_all[:, t:t + 1], k_all[:, t:t + 1], v_all[:, t:t + 1], torch.tensor([t + 1] * B),
                      freqs_cis=freqs, positions=pos, is_prefill=False)
        assert torch.allclose(out_d[:, 0], ref, atol=1e-5), step


def test_double_benchmark_accuracy_criterion():
    """A result as good as the same-precision baseline passes, one that is clearly worse fails, NaN fails."""
    import pytest
    import torch
    from mindformers_b200.utils.precision import DoubleBenchmarkComparator, error_metrics, precision_check
    torch.manual_seed(0)
    a, b = torch.randn(256, 512), torch.randn(512, 128)
    golden = a.double() @ b.double()
    baseline = (a.bfloat16() @ b.bfloat16()).float()
    good = (a.bfloat16().float() @ b.bfloat16().float()).bfloat16().float()          # bf16 inputs, fp32 accumulation
    cmp_ = DoubleBenchmarkComparator(dtype=torch.bfloat16)
    ok, report = cmp_.check_pass_or_not(good, baseline, golden)
    assert ok, report
    worse = good + 0.05 * golden.float().abs().mean() * torch.randn_like(good)
    ok, report = cmp_.check_pass_or_not(worse, baseline, golden)
    assert not ok and not report["rmse"]["passed"]
    broken = good.clone()
    broken[3, 5] = float("nan")
    assert not cmp_.check_pass_or_not(broken, baseline, golden)[0]
    m = error_metrics(good, golden, cmp_.std)
    assert 0 < m["mean_rel"] < 5e-2 and m["rmse"] > 0
    out = precision_check(good, golden.float(), l1_threshold=0.1, kl_threshold=1e-3)
    assert out["cosine"] > 0.9999
    with pytest.raises(AssertionError):
        precision_check(-good, golden.float())


def test_generic_transformer_blocks():
    """Encoder / decoder stacks of the older API: shapes, causal masking, incremental decoding with the returned
    key / value pairs, cross-attention, post- vs pre-LN."""
    import torch
    from mindformers_b200.modules import (AttentionMask, Transformer, TransformerDecoder, TransformerEncoder,
                                          VocabEmbedding)
    torch.manual_seed(0)
    B, S, H = 2, 6, 32
    emb = VocabEmbedding(50, H)
    ids = torch.randint(0, 50, (B, S))
    x, table = emb(ids)
    assert x.shape == (B, S, H) and table.shape == (50, H)
    mask = AttentionMask(S)(torch.tensor([[1, 1, 1, 1, 1, 1], [1, 1, 1, 1, 0, 0]]))
    assert mask.shape == (B, S, S) and mask[0, 2, 3] == 0 and mask[0, 3, 2] == 1 and mask[1, 5, 4] == 0
    enc = TransformerEncoder(B, 2, H, 64, S, 4, 0.0, 0.0, use_past=True).eval()
    full, present = enc(x, mask)
    assert full.shape == (B, S, H) and len(present) == 2 and present[0][0].shape == (B, 4, S, H // 4)
    # causal: a later token does not change earlier outputs
    x2 = x.clone()
    x2[0, 5] += 1.0
    assert torch.allclose(enc(x2, mask)[0][0, :5], full[0, :5], atol=1e-6)
    # incremental: last token with the cached keys / values of the first five
    first, past = enc(x[:, :5], mask[:, :5, :5])
    step, _ = enc(x[:, 5:6], mask[:, 5:6, :], past=past)
    assert torch.allclose(step[0, 0], full[0, 5], atol=1e-5)
    dec = TransformerDecoder(1, B, H, 64, S, 4, 4, 0.0, 0.0, post_layernorm_residual=True).eval()
    tgt = torch.randn(B, 4, H)
    out, _ = dec(tgt, torch.tril(torch.ones(4, 4)).expand(B, 4, 4), full, torch.ones(B, 4, S))
    out_nomem, _ = dec(tgt, torch.tril(torch.ones(4, 4)).expand(B, 4, 4))
    assert out.shape == (B, 4, H) and not torch.allclose(out, out_nomem)
    model = Transformer(H, B, 64, S, 4, encoder_layers=1, decoder_layers=1, num_heads=4, attention_dropout_rate=0.0,
                        hidden_dropout_rate=0.0)
    y, enc_p, dec_p = model(x, mask, tgt, torch.tril(torch.ones(4, 4)).expand(B, 4, 4), torch.ones(B, 4, S))
    assert y.shape == (B, 4, H) and len(enc_p) == 1 and len(dec_p) == 1
    y.sum().backward()
    assert emb.embedding_table.grad is not None


def test_quantization_config_of_a_pretrained_directory_is_applied(tmp_path, monkeypatch):
    """``quantization_config`` in ``config.json`` selects the quantiser when the model is loaded for inference."""
    import json
    import pytest
    import torch
    from mindformers_b200.models import AutoModel
    from mindformers_b200.modules.quantizers import (AutoQuantizationConfig, Fp8BlockConfig, QuantLinear, RtnConfig,
                                                     SmoothQuantConfig)
    assert isinstance(AutoQuantizationConfig.from_dict({"quant_method": "rtn", "weight_dtype": "int4", "x": 1}), RtnConfig)
    assert AutoQuantizationConfig.from_dict({"quant_method": "smoothquant", "alpha": 0.7}).alpha == 0.7
    fp8 = AutoQuantizationConfig.from_dict({"quant_method": "fp8", "fmt": "e4m3", "weight_block_size": [128, 128],
                                            "activation_scheme": "dynamic"})
    assert isinstance(fp8, Fp8BlockConfig) and fp8.weight_block_size == (128, 128)
    assert isinstance(AutoQuantizationConfig.from_dict({"quant_method": "smooth_quant"}), SmoothQuantConfig)
    with pytest.raises(ValueError):
        AutoQuantizationConfig.from_dict({"quant_method": "int3-magic"})
    cfg = dict(model_type="llama", num_hidden_layers=2, hidden_size=128, num_attention_heads=4, num_key_value_heads=2,
               intermediate_size=256, vocab_size=256, max_position_embeddings=64, params_dtype="float32")
    torch.manual_seed(0)
    ref = AutoModel.from_config(cfg, device="cpu").eval()
    ref.save_pretrained(str(tmp_path / "m"))
    saved = json.load(open(tmp_path / "m" / "config.json"))
    saved["quantization_config"] = {"quant_method": "rtn", "weight_dtype": "int8"}
    json.dump(saved, open(tmp_path / "m" / "config.json", "w"))
    monkeypatch.setenv("RUN_MODE", "predict")
    q = AutoModel.from_pretrained(str(tmp_path / "m"), device="cpu").eval()
    n_quant = sum(isinstance(m, QuantLinear) for m in q.modules())
    assert n_quant == 2 * 4                                           # qkv, proj, fc1, fc2 of both layers
    ids = torch.randint(0, 256, (1, 12))
    with torch.no_grad():
        a, b = ref(ids).float(), q(ids).float()
    assert ((a - b).norm() / a.norm()).item() < 0.05
    monkeypatch.setenv("RUN_MODE", "finetune")                        # training keeps full-precision layers
    t = AutoModel.from_pretrained(str(tmp_path / "m"), device="cpu")
    assert not any(isinstance(m, QuantLinear) for m in t.modules())


def test_w8a8_linear_is_exact_integer_arithmetic_and_close_to_the_float_product():
    """Per-token activation scales x per-channel weight scales around an exact integer product."""
    from mindformers_b200.ops import functional as Fn
    torch.manual_seed(31)
    x = torch.randn(37, 96)
    w = torch.randn(40, 96) * 0.1
    wq, ws = Q.quantize_weight_rtn(w, "int8", 0)
    xq, xs = Fn.quantize_act_int8(x)
    assert xq.dtype == torch.int8 and xs.shape == (37,) and int(xq.abs().max()) == 127
    y = Fn.w8a8_gemm(xq, xs, wq, ws[:, 0]).float()
    exact = (xq.double() @ wq.double().t()).float() * xs[:, None] * ws[:, 0][None, :]
    assert torch.allclose(y, exact.to(torch.bfloat16).float())
    ref = x @ w.t()
    assert ((y - ref).norm() / ref.norm()).item() < 0.03
    smooth = torch.rand(96) + 0.5
    y2 = Fn.w8a8_linear(x, Q.quantize_weight_rtn(w * smooth, "int8", 0)[0], Q.quantize_weight_rtn(w * smooth, "int8", 0)[1][:, 0],
                        smooth=smooth)
    assert ((y2.float() - ref).norm() / ref.norm()).item() < 0.03
