"""Block-scaled fp8 inference weights: quantised model close to the bf16 one, generation still runs."""
import torch

from mindformers_b200.inference.fp8 import quantize_model_fp8
from mindformers_b200.models import AutoModel


def tiny_deepseek():
    cfg = dict(model_type="deepseek_v3", num_hidden_layers=3, hidden_size=256, num_attention_heads=4,
               num_key_value_heads=4, intermediate_size=512, moe_intermediate_size=128, n_routed_experts=8,
               n_shared_experts=1, num_experts_per_tok=2, n_group=2, topk_group=1, routed_scaling_factor=1.0,
               norm_topk_prob=True, scoring_func="sigmoid", first_k_dense_replace=1, vocab_size=512,
               q_lora_rank=128, kv_lora_rank=128, qk_nope_head_dim=32, qk_rope_head_dim=16, v_head_dim=32,
               max_position_embeddings=256, params_dtype="float32", moe_router_enable_expert_bias=True)
    torch.manual_seed(0)
    return AutoModel.from_config(cfg, device="cpu").eval()


def test_quantize_model_fp8_matches_full_precision():
    model = tiny_deepseek()
    ids = torch.randint(3, 512, (2, 32))
    with torch.no_grad():
        ref = model(ids).float()
    stats = quantize_model_fp8(model)
    assert stats["linear"] >= 6 and stats["grouped"] == 2 and stats["kept"] >= 1
    assert stats["bytes_after"] < 0.3 * stats["bytes_before"]          # fp32 -> fp8 + scales
    names = dict(model.named_modules())
    dense = names["model.decoder.layers.0.mlp.linear_fc1"]
    assert dense.weight is None and dense.weight_fp8.dtype == torch.float8_e4m3fn
    assert dense.weight_scale_inv.shape == (dense.weight_fp8.shape[0] // 128, dense.weight_fp8.shape[1] // 128)
    assert names["model.output_layer"].weight is not None              # kept in full precision
    with torch.no_grad():
        out = model(ids).float()
    rel = ((out - ref).norm() / ref.norm()).item()
    assert rel < 0.08, rel
    assert (out.argmax(-1) == ref.argmax(-1)).float().mean() > 0.7
    seqs = model.generate(ids[:, :8].tolist(), max_new_tokens=4, do_sample=False)
    assert all(len(s) == 12 for s in seqs)


def test_fp8_checkpoint_roundtrip(tmp_path):
    """A checkpoint with block-scaled fp8 linear weights loads into a model and leaves fp8 layers behind."""
    from safetensors.torch import save_file
    from mindformers_b200.checkpoint import name_maps
    from mindformers_b200.checkpoint.io import load_checkpoint
    model = tiny_deepseek()
    ids = torch.randint(3, 512, (1, 16))
    with torch.no_grad():
        ref = model(ids).float()
    sd = {k: v.detach().clone() for k, v in model.named_parameters()}
    q = name_maps.requantize_linear_weights(sd)
    fp8_names = [k for k, v in q.items() if v.dtype == torch.float8_e4m3fn]
    assert fp8_names and all(k + "_scale_inv" in q for k in fp8_names)
    assert not any("linear_kvb" in k or "router" in k for k in fp8_names)
    # values survive de-quantise -> re-quantise exactly (same blocks, same scales)
    name = fp8_names[0]
    again, scale2 = __import__("mindformers_b200.ops.functional", fromlist=["x"]).quantize_weight_128x128(
        name_maps.weight_dequant(q[name], q[name + "_scale_inv"]).float())
    assert torch.equal(again.view(torch.uint8), q[name].view(torch.uint8))
    save_file({k: v.contiguous() for k, v in q.items()}, str(tmp_path / "model.safetensors"))
    fresh = tiny_deepseek()
    with torch.no_grad():
        for p in fresh.parameters():
            p.add_(1.0)                       # make sure the values come from the file
    load_checkpoint(fresh, str(tmp_path / "model.safetensors"), strict=True, family="deepseek_v3")
    mods = dict(fresh.named_modules())
    assert mods["model.decoder.layers.0.mlp.linear_fc1"].weight_fp8 is not None
    with torch.no_grad():
        out = fresh(ids).float()
    assert ((out - ref).norm() / ref.norm()).item() < 0.08


def test_fp8_linear_with_ragged_output_rows_is_padded_and_sliced():
    """An output width that does not fill its last 128-row block (MLA ``linear_qkv``: q_lora + kv_lora + rope) is
    quantised with zero padding rows; the result has the true width and matches the full-precision layer."""
    model = tiny_deepseek()
    quantize_model_fp8(model)
    lin = dict(model.named_modules())["model.decoder.layers.0.self_attention.linear_qkv"]
    assert lin.weight is None and lin.weight_fp8.shape[0] == 384 and lin._fp8_rows == 128 + 128 + 16
    assert lin.weight_scale_inv.shape == (3, 2)
    ref = tiny_deepseek()
    ref_lin = dict(ref.named_modules())["model.decoder.layers.0.self_attention.linear_qkv"]
    x = torch.randn(5, 256)
    y, y_ref = lin._mm(x), ref_lin._mm(x)
    assert y.shape == y_ref.shape == (5, 272)
    assert ((y.float() - y_ref).norm() / y_ref.norm()).item() < 0.06
