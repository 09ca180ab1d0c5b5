"""Self-attention (MHA/GQA) and multi-latent attention, one implementation for training and inference.

Reference behaviour: ``training_graph/transformer/attention.py`` (QKV projection → split → optional
per-head q/k RMSNorm → RoPE → core attention → output projection, :231-316; contiguous ``[Q;K;V]`` vs
per-group interleaved weight layouts :444,560), ``training_graph/transformer/multi_latent_attention.py``
(:70-342) and the inference modules (``inference/transformer/attention.py`` :214-364,
``inference/transformer/multi_latent_attention.py`` :240-448: latent KV cache ``[kv_lora ‖ k_pe]`` and
weight absorption in decode).

Activations are token-major ``[T, H]``; ``AttnMeta`` says how tokens group into sequences.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn

from ...ops import functional as Fn
from .. import parallel_state as ps
from .norm import RMSNorm, build_norm
from .tensor_parallel import ColumnParallelLinear, LinearNoTP, RowParallelLinear, default_init


@dataclass
class AttnMeta:
    """How the flat token axis maps to sequences for one forward call."""
    batch: int = 1
    seq_len: int = 0                      # tokens per sequence (dense batches)
    positions: Optional[torch.Tensor] = None   # [T] int position ids (None: t % seq_len)
    cu_seqlens: Optional[torch.Tensor] = None  # [n+1] packed-sequence boundaries (TND layout)
    max_seqlen: int = 0
    actual_seq_len: Optional[torch.Tensor] = None   # [B, P] cumulative document ends per row (EOD-reset batches)
    doc_tables: Optional[tuple] = None    # (doc_start, doc_end) int32 [B, S], built once per forward from the above
    cache: Optional[object] = None        # inference.KVCacheContext for paged attention
    kv_carry: Optional[object] = None     # modules.seq_pipe.KVCarry: keys / values of the earlier sequence chunks
    cp_rank_positions: bool = False       # positions already hold the context-parallel offsets


def _local_heads(config):
    tp = ps.get_tensor_model_parallel_world_size()
    nq = config.num_attention_heads // tp
    if config.num_query_groups >= tp:
        nkv = config.num_query_groups // tp
    else:
        nkv = 1  # KV heads are replicated when tp exceeds their number
    return nq, nkv


class CoreAttention(nn.Module):
    """Softmax attention over ``[B, S, heads, hd]`` views; picks dense / context-parallel / paged paths."""

    def __init__(self, config, layer_number: int, softmax_scale: Optional[float] = None, head_dim=None):
        super().__init__()
        self.config = config
        self.layer_number = layer_number
        hd = head_dim or config.kv_channels
        self.scale = softmax_scale if softmax_scale is not None else (config.softmax_scale or 1.0 / math.sqrt(hd))
        self.unfused = None
        if not getattr(config, "use_flash_attention", True):
            from .dot_product_attention import DotProductAttention
            self.unfused = DotProductAttention(config, layer_number, self.scale, hd)

    def forward(self, q, k, v, meta: AttnMeta):
        """q: [T, nq, d]; k: [T, nkv, d]; v: [T, nkv, dv] → [T, nq*dv]."""
        T, nq, _ = q.shape
        if meta.cache is not None:
            from ...inference.paged_attention import paged_attention_forward
            return paged_attention_forward(q, k, v, meta, self.layer_number, self.scale)
        cp = ps.get_context_parallel_world_size()
        B = meta.batch
        S = T // B
        q4, k4, v4 = (t.reshape(B, S, t.shape[1], t.shape[2]) for t in (q, k, v))
        if cp > 1:
            from ..context_parallel import context_parallel_attention
            o = context_parallel_attention(q4, k4, v4, self.scale, self.config)
        elif meta.cu_seqlens is not None or meta.actual_seq_len is not None:
            from ..context_parallel import varlen_attention
            cu = meta.cu_seqlens
            if cu is None:       # cumulative ends per row -> boundaries of the flattened token axis
                ends = meta.actual_seq_len.reshape(B, -1).to(torch.int64).clamp(max=S)
                flat = (ends + torch.arange(B, device=ends.device).unsqueeze(1) * S).reshape(-1)
                cu = torch.unique(torch.cat([flat.new_zeros(1), flat]))
                q4, k4, v4 = (t.reshape(1, B * S, t.shape[2], t.shape[3]) for t in (q4, k4, v4))
            o = varlen_attention(q4, k4, v4, cu, self.scale)
        elif self.unfused is not None:       # use_flash_attention=False: explicit mask + softmax
            o = self.unfused(q4, k4, v4)
        elif self.training and float(getattr(self.config, "attention_dropout", 0.0) or 0.0) > 0.0:
            # dropout on the attention probabilities: the flash kernels have no dropout, the library kernel does
            nq_, nkv_ = q4.shape[2], k4.shape[2]
            o = torch.nn.functional.scaled_dot_product_attention(
                q4.transpose(1, 2), k4.transpose(1, 2), v4.transpose(1, 2), dropout_p=float(self.config.attention_dropout),
                is_causal=True, scale=self.scale, enable_gqa=(nq_ != nkv_)).transpose(1, 2)
        else:
            o = Fn.attention(q4, k4, v4, causal=True, scale=self.scale)
        return o.reshape(T, -1)


class SelfAttention(nn.Module):
    """GQA self-attention with a fused QKV projection.

    Parameter names: ``linear_qkv.{weight,bias}``, ``q_layernorm.weight``, ``k_layernorm.weight``,
    ``linear_proj.weight``. With ``use_contiguous_weight_layout`` the QKV rows are ``[Q; K; V]``;
    otherwise they are interleaved per KV group ``[q×rep, k, v]`` (Megatron layout).
    """

    def __init__(self, config, layer_number: int = 1):
        super().__init__()
        self.config = config
        self.layer_number = layer_number
        self.hd = config.kv_channels
        self.nq_total, self.nkv_total = config.num_attention_heads, config.num_query_groups
        self.nq, self.nkv = _local_heads(config)
        self.contiguous_layout = config.use_contiguous_weight_layout
        q_size, kv_size = self.nq_total * self.hd, self.nkv_total * self.hd
        sections = (q_size, kv_size, kv_size) if self.contiguous_layout else None
        tp = ps.get_tensor_model_parallel_world_size()
        groups = None
        if self.nkv_total < tp:
            # more ranks than KV heads: every rank keeps one whole KV head, replicated over tp / kv_heads ranks
            # (reference: QKVParallelLinear of the inference stack, tensor_parallel/layers.py:262-275). Inference only:
            # the gradients of the replicas are not summed between them.
            if not self.contiguous_layout or tp % self.nkv_total:
                raise NotImplementedError("a tensor-parallel size above the number of KV heads needs the contiguous "
                                          "[Q; K; V] weight layout and tp divisible by the number of KV heads")
            groups = (self.nq_total, self.nkv_total, self.nkv_total)
        self.linear_qkv = ColumnParallelLinear(config.hidden_size, q_size + 2 * kv_size, config=config,
                                               bias=config.add_qkv_bias or config.add_bias_linear,
                                               partition_sections=sections, partition_groups=groups)
        if config.qk_layernorm:
            self.q_layernorm = RMSNorm(config, self.hd, config.layernorm_epsilon)
            self.k_layernorm = RMSNorm(config, self.hd, config.layernorm_epsilon)
        else:
            self.q_layernorm = self.k_layernorm = None
        self.core_attention = CoreAttention(config, layer_number)
        self.linear_proj = RowParallelLinear(q_size, config.hidden_size, config=config,
                                             bias=config.add_bias_linear, skip_bias_add=False)
        self.rot_dim = int(self.hd * config.rotary_percent)

    def _split(self, qkv):
        """[T, local_width] → q [T,nq,hd], k, v [T,nkv,hd] (views when the layout is contiguous)."""
        T = qkv.shape[0]
        if self.contiguous_layout:
            x = qkv.view(T, self.nq + 2 * self.nkv, self.hd)
            return x, x[:, :self.nq], x[:, self.nq:self.nq + self.nkv], x[:, self.nq + self.nkv:]
        rep = self.nq // self.nkv
        g = qkv.view(T, self.nkv, rep + 2, self.hd)
        q = g[:, :, :rep].reshape(T, self.nq, self.hd)
        k, v = g[:, :, rep], g[:, :, rep + 1]
        x = torch.cat((q, k, v), dim=1)
        return x, x[:, :self.nq], x[:, self.nq:self.nq + self.nkv], x[:, self.nq + self.nkv:]

    def forward(self, hidden, rotary, meta: AttnMeta):
        qkv, _ = self.linear_qkv(hidden)
        packed, q, k, v = self._split(qkv)
        if self.q_layernorm is not None:
            qn = self.q_layernorm(q)
            kn = self.k_layernorm(k)
            packed = torch.cat((qn, kn, v), dim=1)
            q, k, v = packed[:, :self.nq], packed[:, self.nq:self.nq + self.nkv], packed[:, self.nq + self.nkv:]
        if rotary is not None:
            cos, sin = rotary
            pos = meta.positions
            if pos is None:
                pos = torch.arange(packed.shape[0], device=packed.device) % max(meta.seq_len, 1)
            packed = Fn.rope(packed if packed.is_contiguous() else packed.contiguous(), cos, sin, pos,
                             self.nq + self.nkv, self.rot_dim, self.config.rotary_interleaved)
            q, k, v = packed[:, :self.nq], packed[:, self.nq:self.nq + self.nkv], packed[:, self.nq + self.nkv:]
        ctx = None
        if meta.kv_carry is not None:
            # sequence pipeline: this call holds one chunk of every sequence; attend to the chunks before it as well
            carry = meta.kv_carry
            T = packed.shape[0]
            B, S = meta.batch, T // meta.batch
            k4, v4 = k.reshape(B, S, self.nkv, self.hd), v.reshape(B, S, self.nkv, self.hd)
            k_all, v_all = carry.extend(self.layer_number, k4, v4)
            q4 = q.reshape(B, S, self.nq, self.hd)
            from ...ops import attention as native
            if k_all.shape[1] == S:
                o = Fn.attention(q4, k_all, v_all, causal=True, scale=self.core_attention.scale)
            elif native.rect_supported(q4, k_all, v_all) and Fn.get_attention_backend() != "sdpa":
                o = native.flash_attention_rect(q4.contiguous(), k_all.contiguous(), v_all.contiguous(), carry.start, True,
                                                self.core_attention.scale)
            else:
                o = Fn.attention_reference(q4, k_all, v_all, True, self.core_attention.scale, q_offset=carry.start)
            ctx = o.reshape(T, self.nq * self.hd)
        drop = self.training and float(getattr(self.config, "attention_dropout", 0.0) or 0.0) > 0.0
        if ctx is None and meta.cache is None and ps.get_context_parallel_world_size() == 1 and not drop \
                and Fn.get_attention_backend() != "sdpa" and getattr(self, "use_packed_attention", True):
            from ...ops import attention as native
            T = packed.shape[0]
            S = T // meta.batch
            if native.packed_supported(packed, S, self.nq, self.nkv):
                docs = (None, None)
                if meta.cu_seqlens is not None or meta.actual_seq_len is not None:
                    # packed rows (EOD-reset data, TND batches): the kernels take per-token document tables
                    if meta.doc_tables is None:
                        meta.doc_tables = native.document_tables(meta.cu_seqlens, meta.actual_seq_len, meta.batch, S)
                    docs = meta.doc_tables
                ctx = native.flash_attention_packed(packed, meta.batch, S, self.nq, self.nkv, True,
                                                    self.core_attention.scale, docs[0], docs[1])
        if ctx is None:
            ctx = self.core_attention(q, k, v, meta)
        out, bias = self.linear_proj(ctx)
        return out, bias


class MLASelfAttention(nn.Module):
    """Multi-latent attention (DeepSeek-V2/V3).

    Training layout (``mla_qkv_concat``): ``linear_qkv`` = [q_down ‖ kv_down ‖ k_pe] (replicated),
    ``q_layernorm``, ``linear_qb`` (q up, column-parallel), ``kv_layernorm`` (``k_layernorm``),
    ``linear_kvb`` (kv up, column-parallel), ``linear_proj``. Without ``q_lora_rank`` the query is a plain
    column-parallel ``linear_q``. Decode with a paged cache stores ``[kv_lora ‖ k_pe]`` per token and
    absorbs the up-projections into q and the output.
    """

    def __init__(self, config, layer_number: int = 1):
        super().__init__()
        self.config = config
        self.layer_number = layer_number
        tp = ps.get_tensor_model_parallel_world_size()
        self.nh = config.num_attention_heads // tp
        self.nope, self.rope_d, self.vd = config.qk_head_dim, config.qk_pos_emb_head_dim, config.v_head_dim
        self.qd = self.nope + self.rope_d
        self.q_rank, self.kv_rank = config.q_lora_rank, config.kv_lora_rank
        H = config.hidden_size
        replicated = self._build_projections(config, H)
        self.linear_proj = RowParallelLinear(config.num_attention_heads * self.vd, H, config=config,
                                             bias=config.add_bias_linear)
        # these run on the gathered sequence: their gradients are already complete on every rank
        for mod in replicated:
            if mod is not None:
                for prm in mod.parameters():
                    prm.sequence_parallel = False
        mscale = 1.0
        if config.rope_type == "yarn" and config.rotary_scaling_factor > 1 and config.mscale_all_dim:
            from .rotary import yarn_get_mscale
            mscale = yarn_get_mscale(config.rotary_scaling_factor, config.mscale_all_dim)
        self.scale = config.softmax_scale or (mscale * mscale / math.sqrt(self.qd))
        self.core_attention = CoreAttention(config, layer_number, softmax_scale=self.scale, head_dim=self.qd)

    def _build_projections(self, config, H):
        """Create the query / kv projections and norms; returns the modules that run replicated on the full sequence."""
        down = (self.q_rank or 0) + self.kv_rank + self.rope_d
        if self.q_rank:
            self.linear_qkv = LinearNoTP(H, down, config=config)
            self.q_layernorm = RMSNorm(config, self.q_rank, config.layernorm_epsilon)
            self.linear_qb = ColumnParallelLinear(self.q_rank, config.num_attention_heads * self.qd, config=config)
        else:
            self.linear_q = ColumnParallelLinear(H, config.num_attention_heads * self.qd, config=config)
            self.linear_qkv = LinearNoTP(H, down, config=config)
            self.q_layernorm = None
        self.k_layernorm = RMSNorm(config, self.kv_rank, config.layernorm_epsilon)
        self.linear_kvb = ColumnParallelLinear(self.kv_rank, config.num_attention_heads * (self.nope + self.vd),
                                               config=config)
        return self.linear_qkv, self.q_layernorm, self.k_layernorm

    def _rope(self, x, rotary, meta, heads):
        cos, sin = rotary
        pos = meta.positions
        if pos is None:
            pos = torch.arange(x.shape[0], device=x.device) % max(meta.seq_len, 1)
        return Fn.rope(x.contiguous(), cos, sin, pos, heads, self.rope_d, self.config.rotary_interleaved)

    def forward(self, hidden, rotary, meta: AttnMeta):
        sp_gather = self.config.sequence_parallel and ps.get_tensor_model_parallel_world_size() > 1
        if sp_gather:
            from .. import mappings as M
            # every rank then runs the replicated projections on the full sequence, so the gradient
            # of this gather is a plain split (the column-parallel branches all-reduce theirs first)
            hidden_full = M.gather_from_sequence_parallel_region(hidden, reduce_scatter_grad=False)
        else:
            hidden_full = hidden
        T = hidden_full.shape[0]
        q, kv_c, k_pe = self._project(hidden_full)
        q = q.view(T, self.nh, self.qd)
        q_nope, q_pe = q[..., :self.nope], q[..., self.nope:]
        kv_c = self.k_layernorm(kv_c)
        q_pe = self._rope(q_pe, rotary, meta, self.nh)
        k_pe = self._rope(k_pe.reshape(T, 1, self.rope_d), rotary, meta, 1)
        if meta.cache is not None:
            from ...inference.paged_attention import mla_paged_attention_forward
            ctx = mla_paged_attention_forward(self, q_nope, q_pe, kv_c, k_pe, meta)
        else:
            kv = self._col_nosp(self.linear_kvb, kv_c).view(T, self.nh, self.nope + self.vd)
            k_nope, v = kv[..., :self.nope], kv[..., self.nope:]
            k = torch.cat((k_nope, k_pe.expand(T, self.nh, self.rope_d)), dim=-1)
            qf = torch.cat((q_nope, q_pe), dim=-1)
            if self.vd != self.qd:
                v = torch.nn.functional.pad(v, (0, self.qd - self.vd))
            ctx = self.core_attention(qf, k, v, meta).view(T, self.nh, self.qd)[..., :self.vd].reshape(T, -1)
        out, bias = self.linear_proj(ctx)
        return out, bias

    def _project(self, hidden_full):
        """Full-sequence hidden states → (query ``[T, nh·qd]``, compressed kv ``[T, kv_rank]``, shared rotary key
        ``[T, rope_d]``), before the kv norm and the rotary embedding."""
        comp, _ = self.linear_qkv(hidden_full)
        if self.q_rank:
            q_c, kv_c, k_pe = torch.split(comp, [self.q_rank, self.kv_rank, self.rope_d], dim=-1)
            q = self._col_nosp(self.linear_qb, self.q_layernorm(q_c))
        else:
            kv_c, k_pe = torch.split(comp, [self.kv_rank, self.rope_d], dim=-1)
            q = self._col_nosp(self.linear_q, hidden_full)
        return q, kv_c, k_pe

    def _col_nosp(self, layer, x):
        """Column-parallel projection of an input that is already full-sequence on every rank."""
        if layer.tp > 1:
            from .. import mappings as M
            x = M.copy_to_tensor_model_parallel_region(x)
        y = layer._mm(x)
        if layer.bias is not None:
            y = y + layer.bias
        return y


class MLASelfAttentionMegatron(MLASelfAttention):
    """Multi-latent attention with one module per projection, under the names Megatron checkpoints use
    (reference ``training_graph/transformer/multi_latent_attention.py:345-520``, selected by
    ``mla_qkv_concat=False``): ``linear_q_proj`` (no query compression) or ``linear_q_down_proj`` → ``q_layernorm``
    → ``linear_q_up_proj``; ``linear_kv_down_proj`` (``[kv_lora ‖ k_pe]``) → ``kv_layernorm`` →
    ``linear_kv_up_proj``; ``linear_proj``. The arithmetic, the paged decode path and the weight absorption are those
    of ``MLASelfAttention``; only the parameter layout differs, so a checkpoint in this layout loads without the
    down-projections being concatenated."""

    def _build_projections(self, config, H):
        nhq = config.num_attention_heads * self.qd
        if self.q_rank:
            self.linear_q_down_proj = LinearNoTP(H, self.q_rank, config=config)
            self.q_layernorm = RMSNorm(config, self.q_rank, config.layernorm_epsilon)
            self.linear_q_up_proj = ColumnParallelLinear(self.q_rank, nhq, config=config)
        else:
            self.linear_q_proj = ColumnParallelLinear(H, nhq, config=config)
            self.q_layernorm = None
        self.linear_kv_down_proj = LinearNoTP(H, self.kv_rank + self.rope_d, config=config)
        self.kv_layernorm = RMSNorm(config, self.kv_rank, config.layernorm_epsilon)
        self.linear_kv_up_proj = ColumnParallelLinear(self.kv_rank, config.num_attention_heads * (self.nope + self.vd),
                                                      config=config)
        return (getattr(self, "linear_q_down_proj", None), self.linear_kv_down_proj, self.q_layernorm,
                self.kv_layernorm)

    # the shared forward and the paged decode path address the kv norm and up-projection by the concatenated
    # layout's names
    @property
    def k_layernorm(self):
        return self.kv_layernorm

    @property
    def linear_kvb(self):
        return self.linear_kv_up_proj

    def _project(self, hidden_full):
        kv, _ = self.linear_kv_down_proj(hidden_full)
        kv_c, k_pe = torch.split(kv, [self.kv_rank, self.rope_d], dim=-1)
        if self.q_rank:
            q_c, _ = self.linear_q_down_proj(hidden_full)
            q = self._col_nosp(self.linear_q_up_proj, self.q_layernorm(q_c))
        else:
            q = self._col_nosp(self.linear_q_proj, hidden_full)
        return q, kv_c, k_pe


class CrossAttention(nn.Module):
    """Attention whose queries come from the layer input and whose keys and values come from another sequence
    (an encoder's output): ``linear_q`` (hidden → heads·hd, column-parallel), ``linear_kv`` (hidden → 2·heads·hd,
    column-parallel, rows ``[K; V]`` per rank), non-causal softmax attention, ``linear_proj`` (row-parallel).
    Reference ``training_graph/transformer/attention.py:670-760``: like there, the number of query groups must equal
    the number of heads, and no rotary embedding is applied.

    ``forward(hidden [Tq, H], key_value_states [Tk, H], meta, kv_batch_seq=None)``: both inputs are token-major with
    ``meta.batch`` sequences of equal length each."""

    def __init__(self, config, layer_number: int = 1):
        super().__init__()
        if config.num_query_groups != config.num_attention_heads:
            raise ValueError("cross attention needs num_query_groups == num_attention_heads")
        self.config, self.layer_number = config, layer_number
        self.hd = config.kv_channels
        tp = ps.get_tensor_model_parallel_world_size()
        self.nh = config.num_attention_heads // tp
        width = config.num_attention_heads * self.hd
        bias = config.add_qkv_bias or config.add_bias_linear
        self.linear_q = ColumnParallelLinear(config.hidden_size, width, config=config, bias=bias)
        self.linear_kv = ColumnParallelLinear(config.hidden_size, 2 * width, config=config, bias=bias,
                                              partition_sections=(width, width))
        self.linear_proj = RowParallelLinear(width, config.hidden_size, config=config, bias=config.add_bias_linear,
                                             skip_bias_add=False)
        self.scale = config.softmax_scale or 1.0 / math.sqrt(self.hd)

    def forward(self, hidden, key_value_states, meta: AttnMeta, rotary=None):
        q, _ = self.linear_q(hidden)
        kv, _ = self.linear_kv(key_value_states)
        B = meta.batch
        Tq, Tk = q.shape[0], kv.shape[0]
        q4 = q.view(B, Tq // B, self.nh, self.hd)
        kv5 = kv.view(B, Tk // B, 2, self.nh, self.hd)
        o = Fn.attention(q4, kv5[:, :, 0], kv5[:, :, 1], causal=False, scale=self.scale)
        return self.linear_proj(o.reshape(Tq, self.nh * self.hd))
