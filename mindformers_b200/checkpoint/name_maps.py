"""Hugging Face ⇄ framework parameter names and layouts.

Step 1 renames HF keys to per-projection framework names (the maps of the reference's
``models/qwen3/utils.py:31-64``, ``models/qwen2/utils.py:30-57``, ``models/deepseek3/utils.py:32-71``,
``models/llama/llama.py:682-702``). Step 2 fuses them into the parameters the network owns
(``inference/model_utils.py:83-114``, ``toolkit/weight_convert/deepseekv3/convert_deepseekv3_hf_weight.py``):

* ``linear_q | linear_k | linear_v``  → ``linear_qkv``  (rows ``[Q; K; V]``, or per-KV-group interleave)
* ``mlp.gating | mlp.linear_fc1``     → ``mlp.linear_fc1`` (rows ``[gate; up]``)
* ``experts.N.{gating,linear_fc1}``   → ``experts.weight1`` ``[E, H, 2F]``;  ``experts.N.linear_fc2`` → ``weight2 [E, F, H]``
* MLA: ``linear_q_down_proj | linear_kv_down_proj`` → ``linear_qkv``; ``linear_q_up_proj`` → ``linear_qb``;
  ``linear_kv_up_proj`` → ``linear_kvb``; ``kv_layernorm`` → ``k_layernorm``
* ``router.weight.weight`` → ``router.weight``
"""
from __future__ import annotations

import re
from typing import Dict, List, Optional, Tuple

import torch

_COMMON = [
    ("model.embed_tokens.", "embedding.word_embeddings."),
    (".self_attn.q_proj.", ".self_attention.linear_q."),
    (".self_attn.k_proj.", ".self_attention.linear_k."),
    (".self_attn.v_proj.", ".self_attention.linear_v."),
    (".self_attn.o_proj.", ".self_attention.linear_proj."),
    (".self_attn.q_norm.", ".self_attention.q_layernorm."),
    (".self_attn.k_norm.", ".self_attention.k_layernorm."),
    (".self_attn.q_a_proj.", ".self_attention.linear_q_down_proj."),
    (".self_attn.q_a_layernorm.", ".self_attention.q_layernorm."),
    (".self_attn.q_b_proj.", ".self_attention.linear_q_up_proj."),
    (".self_attn.kv_a_proj_with_mqa.", ".self_attention.linear_kv_down_proj."),
    (".self_attn.kv_a_layernorm.", ".self_attention.kv_layernorm."),
    (".self_attn.kv_b_proj.", ".self_attention.linear_kv_up_proj."),
    (".mlp.shared_expert_gate.weight", ".mlp.shared_experts.gate_weight"),        # Qwen2-MoE: gated shared expert
    (".mlp.shared_expert.", ".mlp.shared_experts."),
    (".mlp.gate.e_score_correction_bias", ".mlp.router.expert_bias"),
    (".mlp.gate.weight", ".mlp.router.weight.weight"),
    (".gate_proj.", ".gating."),
    (".down_proj.", ".linear_fc2."),
    (".up_proj.", ".linear_fc1."),
    (".post_attention_layernorm.", ".pre_mlp_layernorm."),
    ("model.norm.", "decoder.final_layernorm."),
    ("lm_head.", "output_layer."),
    ("model.layers.", "decoder.layers."),
]

# legacy (use_legacy: True) Llama names of the reference: models/llama/llama.py:682-702
_LEGACY_LLAMA = [
    ("model.embed_tokens.weight", "model.tok_embeddings.embedding_weight"),
    (".self_attn.q_proj.", ".attention.wq."),
    (".self_attn.k_proj.", ".attention.wk."),
    (".self_attn.v_proj.", ".attention.wv."),
    (".self_attn.o_proj.", ".attention.wo."),
    (".mlp.gate_proj.", ".feed_forward.w1."),
    (".mlp.down_proj.", ".feed_forward.w2."),
    (".mlp.up_proj.", ".feed_forward.w3."),
    (".input_layernorm.", ".attention_norm."),
    (".post_attention_layernorm.", ".ffn_norm."),
    ("model.norm.", "model.norm_out."),
]

# ChatGLM2/3 and GLM-4 checkpoints (Hugging Face ``THUDM/glm-4-9b`` key names, which the reference's GLM model keeps:
# models/glm2/convert_weight.py:60-160). ``query_key_value`` rows are ``[Q; K; V]`` and ``dense_h_to_4h`` rows are
# ``[gate; up]``: the fused layouts of ``linear_qkv`` and ``linear_fc1``, so they map without splitting. The second
# block covers the reference's split MindSpore names (``qkv_concat`` / ``mlp_concat`` off).
_GLM = [
    ("transformer.embedding.word_embeddings.", "embedding.word_embeddings."),
    ("transformer.embedding.embedding_weight", "embedding.word_embeddings.weight"),
    ("transformer.encoder.final_layernorm.", "decoder.final_layernorm."),
    ("transformer.encoder.layers.", "decoder.layers."),
    ("transformer.output_layer.", "output_layer."),
    (".self_attention.query_key_value.", ".self_attention.linear_qkv."),
    (".self_attention.dense.", ".self_attention.linear_proj."),
    (".mlp.dense_h_to_4h.", ".mlp.linear_fc1."),
    (".mlp.dense_4h_to_h.", ".mlp.linear_fc2."),
    (".post_attention_layernorm.", ".pre_mlp_layernorm."),
]
_GLM_SPLIT = [
    (".self_attention.wq.", ".self_attention.linear_q."),
    (".self_attention.wk.", ".self_attention.linear_k."),
    (".self_attention.wv.", ".self_attention.linear_v."),
    (".mlp.dense_left.", ".mlp.gating."),
    (".mlp.dense_right.", ".mlp.linear_fc1."),
]


def is_glm_name(name: str) -> bool:
    return name.startswith("transformer.")


def convert_name_glm(name: str) -> str:
    """ChatGLM / GLM-4 key → framework key (fused ``linear_qkv`` / ``linear_fc1`` names for the concatenated tensors,
    per-projection names for the split ones)."""
    out = name
    for a, b in _GLM_SPLIT + _GLM:
        out = out.replace(a, b)
    return out


def reverse_name_glm(name: str) -> str:
    """Framework key (fused names) → ChatGLM / GLM-4 key."""
    out = name
    for a, b in _GLM:
        if not a.endswith("embedding_weight"):        # the reference's MindSpore-only spelling: read, never written
            out = out.replace(b, a)
    return out


FAMILIES = ("llama", "qwen2", "qwen2_5", "qwen2_moe", "qwen3", "qwen3_moe", "deepseek_v2", "deepseek_v3",
            "deepseekv3", "mixtral", "telechat", "glm")


def convert_name(hf_name: str, family: str = "llama") -> str:
    """HF key → per-projection framework key."""
    if family == "glm" and is_glm_name(hf_name):
        return convert_name_glm(hf_name)
    out = hf_name
    for a, b in _COMMON:
        out = out.replace(a, b)
    return out


def convert_name_legacy(hf_name: str) -> str:
    out = hf_name
    for a, b in _LEGACY_LLAMA:
        out = out.replace(a, b)
    return out


_LEGACY_MARKS = (".attention.wq.", ".attention.wk.", ".attention.wv.", ".attention.wo.", ".attention.w_qkv.",
                 ".feed_forward.w", "tok_embeddings.", ".attention_norm.", ".ffn_norm.", "model.norm_out.")


def is_legacy_llama_name(name: str) -> bool:
    return any(m in name for m in _LEGACY_MARKS)


def legacy_llama_to_hf_name(name: str) -> str:
    """Legacy Llama key → Hugging Face key (the inverse of ``convert_name_legacy``); the fused ``w_qkv`` /
    ``w_gate_hidden`` keys have no Hugging Face spelling and are handled by ``legacy_llama_to_framework``."""
    out = name
    for hf, legacy in _LEGACY_LLAMA:
        out = out.replace(legacy, hf)
    return out


def legacy_llama_to_framework(sd: Dict[str, torch.Tensor], config) -> Dict[str, torch.Tensor]:
    """State dict with the reference's legacy Llama names → fused framework names. ``attention.w_qkv`` (rows
    ``[Q; K; V]``) and ``feed_forward.w_gate_hidden`` (rows ``[gate; up]``) are the fused layouts already."""
    direct: Dict[str, torch.Tensor] = {}
    per_proj: Dict[str, torch.Tensor] = {}
    for name, t in sd.items():
        if ".attention.w_qkv." in name:
            new = name.replace("model.layers.", "decoder.layers.").replace(".attention.w_qkv.", ".self_attention.linear_qkv.")
            direct[new] = t
        elif ".feed_forward.w_gate_hidden." in name:
            new = name.replace("model.layers.", "decoder.layers.").replace(".feed_forward.w_gate_hidden.", ".mlp.linear_fc1.")
            direct[new] = t
        else:
            per_proj[convert_name(legacy_llama_to_hf_name(name))] = t
    out = fuse_state_dict(per_proj, config)
    out.update(direct)
    return out


def framework_to_legacy_llama(sd: Dict[str, torch.Tensor], config, qkv_concat: bool = False) -> Dict[str, torch.Tensor]:
    """Fused framework names → the reference's legacy Llama names; slices are views of the fused tensors."""
    out: Dict[str, torch.Tensor] = {}
    fused = {}
    if qkv_concat:
        for name in list(sd):
            if name.endswith((".self_attention.linear_qkv.weight", ".self_attention.linear_qkv.bias")):
                new = name.replace("decoder.layers.", "model.layers.").replace(".self_attention.linear_qkv.", ".attention.w_qkv.")
                fused[name] = new
            elif re.search(r"\.mlp\.linear_fc1\.(weight|bias)$", name):
                new = name.replace("decoder.layers.", "model.layers.").replace(".mlp.linear_fc1.", ".feed_forward.w_gate_hidden.")
                fused[name] = new
    rest = {k: v for k, v in sd.items() if k not in fused}
    for name, t in unfuse_state_dict(rest, config).items():
        out[convert_name_legacy(reverse_name(name))] = t
    for name, new in fused.items():
        out[new] = sd[name]
    return out


def reverse_name(mf_name: str) -> str:
    """Per-projection framework key → HF key."""
    out = mf_name
    for a, b in reversed(_COMMON):
        out = out.replace(b, a)
    return out


def qkv_concat(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, num_heads: int, num_kv_heads: int,
               contiguous_layout: bool = True) -> torch.Tensor:
    """Fuse q/k/v weights (rows) or biases. ``contiguous_layout`` gives ``[Q; K; V]``; otherwise the rows are
    interleaved per KV group as ``[q×rep, k, v]`` (reference ``utils/convert_utils.py:63-92``)."""
    if contiguous_layout:
        return torch.cat((q, k, v), dim=0)
    hd = q.shape[0] // num_heads
    rep = num_heads // num_kv_heads
    tail = q.shape[1:]
    qg = q.reshape(num_kv_heads, rep * hd, *tail)
    kg = k.reshape(num_kv_heads, hd, *tail)
    vg = v.reshape(num_kv_heads, hd, *tail)
    return torch.cat((qg, kg, vg), dim=1).reshape(-1, *tail)


def qkv_split(qkv: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int, contiguous_layout: bool = True):
    if contiguous_layout:
        return torch.split(qkv, [num_heads * head_dim, num_kv_heads * head_dim, num_kv_heads * head_dim], dim=0)
    rep = num_heads // num_kv_heads
    tail = qkv.shape[1:]
    g = qkv.reshape(num_kv_heads, (rep + 2) * head_dim, *tail)
    q = g[:, : rep * head_dim].reshape(-1, *tail)
    k = g[:, rep * head_dim:(rep + 1) * head_dim].reshape(-1, *tail)
    v = g[:, (rep + 1) * head_dim:].reshape(-1, *tail)
    return q, k, v


_EXPERT_RE = re.compile(r"^(?P<pre>.*\.mlp\.experts)\.(?P<idx>\d+)\.(?P<proj>gating|linear_fc1|linear_fc2)\.weight$")


def fuse_state_dict(sd: Dict[str, torch.Tensor], config) -> Dict[str, torch.Tensor]:
    """Per-projection framework names → the fused parameters of ``GPTModel`` (full, unsharded tensors)."""
    out: Dict[str, torch.Tensor] = {}
    nh, nkv = config.num_attention_heads, config.num_query_groups
    contiguous = getattr(config, "use_contiguous_weight_layout", True)
    groups: Dict[str, Dict[str, torch.Tensor]] = {}
    experts: Dict[str, Dict[Tuple[int, str], torch.Tensor]] = {}
    # a model built with one module per MLA projection keeps the per-projection names as they are
    split_mla = bool(getattr(config, "multi_latent_attention", False)) and not getattr(config, "mla_qkv_concat", True)
    pats = [r"(.*\.self_attention)\.linear_(q|k|v)\.(weight|bias)$",
            r"(.*\.(?:mlp|shared_experts))\.(gating|linear_fc1)\.(weight|bias)$"]
    if not split_mla:
        pats.append(r"(.*\.self_attention)\.linear_(q_down_proj|kv_down_proj)\.(weight)$")
    for name, t in sd.items():
        m = _EXPERT_RE.match(name)
        if m:
            experts.setdefault(m["pre"], {})[(int(m["idx"]), m["proj"])] = t
            continue
        key = None
        for pat in pats:
            mm = re.match(pat, name)
            if mm:
                key = (mm.group(1), mm.group(3), pat)
                groups.setdefault(str(key), {"_key": key})[mm.group(2)] = t
                break
        if key is not None:
            continue
        new = name
        new = new.replace(".router.weight.weight", ".router.weight")
        if not split_mla:
            new = new.replace(".self_attention.linear_q_up_proj.", ".self_attention.linear_qb.")
            new = new.replace(".self_attention.linear_q_proj.", ".self_attention.linear_q.")
            new = new.replace(".self_attention.linear_kv_up_proj.", ".self_attention.linear_kvb.")
            new = new.replace(".self_attention.kv_layernorm.", ".self_attention.k_layernorm.")
        out[new] = t
    for g in groups.values():
        prefix, kind, _ = g["_key"]
        if "q" in g and "k" in g and "v" in g:
            out[f"{prefix}.linear_qkv.{kind}"] = qkv_concat(g["q"], g["k"], g["v"], nh, nkv, contiguous)
        elif "gating" in g and "linear_fc1" in g:
            out[f"{prefix}.linear_fc1.{kind}"] = torch.cat((g["gating"], g["linear_fc1"]), dim=0)
        elif "kv_down_proj" in g:
            parts = [g["q_down_proj"]] if "q_down_proj" in g else []
            out[f"{prefix}.linear_qkv.{kind}"] = torch.cat(parts + [g["kv_down_proj"]], dim=0)
        else:
            for k2, t in g.items():
                if k2 != "_key":
                    name = {"q": "linear_q_proj" if split_mla else "linear_q", "k": "linear_k", "v": "linear_v"}.get(k2, k2)
                    out[f"{prefix}.{name}.{kind}"] = t
    for prefix, items in experts.items():
        n = max(i for i, _ in items) + 1
        w1 = [torch.cat((items[(e, "gating")], items[(e, "linear_fc1")]), dim=0).t() for e in range(n)]
        w2 = [items[(e, "linear_fc2")].t() for e in range(n)]
        out[f"{prefix}.weight1"] = torch.stack(w1).contiguous()     # [E, H, 2F]
        out[f"{prefix}.weight2"] = torch.stack(w2).contiguous()     # [E, F, H]
    return out


def unfuse_state_dict(sd: Dict[str, torch.Tensor], config) -> Dict[str, torch.Tensor]:
    """Inverse of ``fuse_state_dict`` (used by the reversed converter)."""
    out: Dict[str, torch.Tensor] = {}
    nh, nkv = config.num_attention_heads, config.num_query_groups
    hd = getattr(config, "kv_channels", None) or config.hidden_size // nh
    contiguous = getattr(config, "use_contiguous_weight_layout", True)
    mla = bool(getattr(config, "multi_latent_attention", False))
    for name, t in sd.items():
        if name.endswith((".self_attention.linear_qkv.weight", ".self_attention.linear_qkv.bias")):
            prefix, kind = name.rsplit(".linear_qkv.", 1)
            if mla:
                qr = getattr(config, "q_lora_rank", None) or 0
                if qr:
                    out[f"{prefix}.linear_q_down_proj.{kind}"] = t[:qr]
                out[f"{prefix}.linear_kv_down_proj.{kind}"] = t[qr:]
            else:
                q, k, v = qkv_split(t, nh, nkv, hd, contiguous)
                out[f"{prefix}.linear_q.{kind}"], out[f"{prefix}.linear_k.{kind}"], out[f"{prefix}.linear_v.{kind}"] = q, k, v
        elif re.search(r"\.(mlp|shared_experts)\.linear_fc1\.(weight|bias)$", name) and getattr(config, "gated_linear_unit", True):
            prefix, kind = name.rsplit(".linear_fc1.", 1)
            g, u = t.chunk(2, dim=0)
            out[f"{prefix}.gating.{kind}"], out[f"{prefix}.linear_fc1.{kind}"] = g, u
        elif name.endswith(".experts.weight1"):
            prefix = name[: -len(".weight1")]
            for e in range(t.shape[0]):
                g, u = t[e].t().chunk(2, dim=0)
                out[f"{prefix}.{e}.gating.weight"], out[f"{prefix}.{e}.linear_fc1.weight"] = g.contiguous(), u.contiguous()
        elif name.endswith(".experts.weight2"):
            prefix = name[: -len(".weight2")]
            for e in range(t.shape[0]):
                out[f"{prefix}.{e}.linear_fc2.weight"] = t[e].t().contiguous()
        else:
            new = name.replace(".self_attention.linear_qb.", ".self_attention.linear_q_up_proj.")
            new = new.replace(".self_attention.linear_kvb.", ".self_attention.linear_kv_up_proj.")
            if mla:
                new = new.replace(".self_attention.k_layernorm.", ".self_attention.kv_layernorm.")
            if new.endswith(".router.weight"):
                new = new + ".weight"
            out[new] = t
    return out


def weight_dequant(weight: torch.Tensor, scale_inv: torch.Tensor, block: int = 128) -> torch.Tensor:
    """Block-scaled fp8 (e4m3) weight ``[M, N]`` with fp32 ``scale_inv [ceil(M/128), ceil(N/128)]`` → bf16."""
    M, N = weight.shape
    s = scale_inv.float().repeat_interleave(block, dim=0)[:M].repeat_interleave(block, dim=1)[:, :N]
    return (weight.float() * s).to(torch.bfloat16)


def hf_to_framework(hf_sd: Dict[str, torch.Tensor], config, family: str = "llama", dtype=None,
                    keep_fp8: bool = False) -> Dict[str, torch.Tensor]:
    """Full conversion of an HF state dict (fp8 block-scaled weights are dequantised unless ``keep_fp8``)."""
    plain: Dict[str, torch.Tensor] = {}
    any_fp8 = False
    for name, t in hf_sd.items():
        if name.endswith("_scale_inv"):
            continue
        if t.dtype == torch.float8_e4m3fn:
            sc = hf_sd.get(name + "_scale_inv")
            if sc is None:
                raise KeyError(f"{name} is fp8 but {name}_scale_inv is missing")
            t = weight_dequant(t, sc)           # the fused layouts are built from full-precision tensors
            any_fp8 = True
        if "rotary_emb.inv_freq" in name or "rotary_pos_emb.inv_freq" in name:
            continue
        if dtype is not None and t.is_floating_point():
            t = t.to(dtype)
        plain[convert_name(name, family)] = t
    out = fuse_state_dict(plain, config)
    if keep_fp8 and any_fp8:
        out = requantize_linear_weights(out)
    return out


FP8_KEEP_FULL_PRECISION = ("embedding", "output_layer", "router", "linear_kvb", "layernorm", "norm")


def requantize_linear_weights(sd: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """Fused 2-D ``linear_*`` weights back to block-scaled fp8: ``X.weight`` (e4m3) + ``X.weight_scale_inv`` (fp32, one
    per 128 x 128 block). Blocks of the fused tensors coincide with the blocks of their fp8 sources whenever the
    fused parts are multiples of 128 rows, so the values survive the round trip. Weights whose shape is not a
    multiple of 128, expert stacks and the layers in ``FP8_KEEP_FULL_PRECISION`` stay as they are."""
    from ..ops.functional import quantize_weight_128x128
    out: Dict[str, torch.Tensor] = {}
    for name, t in sd.items():
        if (name.endswith(".weight") and t.dim() == 2 and ".linear_" in name and t.shape[0] % 128 == 0
                and t.shape[1] % 128 == 0 and not any(k in name for k in FP8_KEEP_FULL_PRECISION)):
            q, scale = quantize_weight_128x128(t)
            out[name] = q
            out[name + "_scale_inv"] = scale
        else:
            out[name] = t
    return out


def framework_to_hf(sd: Dict[str, torch.Tensor], config, family: str = "llama", dtype=None) -> Dict[str, torch.Tensor]:
    out = {}
    if family == "glm":       # GLM checkpoints keep the fused query_key_value / dense_h_to_4h tensors
        for name, t in sd.items():
            if dtype is not None and t.is_floating_point():
                t = t.to(dtype)
            out[reverse_name_glm(name)] = t.contiguous()
        return out
    for name, t in unfuse_state_dict(sd, config).items():
        if dtype is not None and t.is_floating_point():
            t = t.to(dtype)
        out[reverse_name(name)] = t.contiguous()
    return out
