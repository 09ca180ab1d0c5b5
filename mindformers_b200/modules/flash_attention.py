"""``FlashAttention`` layer with the reference's call signature (reference ``modules/flash_attention.py:25``).

``forward(query, key, value, attn_mask=None, alibi_mask=None, padding_mask=None, prefix=None, actual_seq_qlen=None,
actual_seq_kvlen=None)`` with ``input_layout`` "BSH" (``[B, S, heads * D]``), "BNSD" (``[B, heads, S, D]``) or "TH"
(packed tokens ``[T, heads * D]`` with cumulative ``actual_seq_*len``). ``attn_mask`` follows the reference's
convention: 1 = discard. The causal cases (``sparse_mode`` 2 / 3 without an explicit mask or alibi) run the
tcgen05 flash-attention kernel through ``ops.functional.attention``; explicit masks, alibi biases, bands
(``sparse_mode`` 4 with ``pre_tokens`` / ``next_tokens``) and dropout take the dense fp32 path."""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from ..ops import functional as Fn

_INT_MAX = 2147483647


class FlashAttention(nn.Module):
    def __init__(self, head_num: int, keep_prob: float = 1.0, scale_value: float = 1.0, pre_tokens: int = _INT_MAX,
                 next_tokens: int = _INT_MAX, input_layout: str = "BSH", sparse_mode: int = 0, use_attention_mask: bool = True,
                 use_alibi_mask: bool = False, use_mqa: bool = False, use_actual_seqlen: bool = False, dp: int = 1, mp: int = 1,
                 cp: int = 1, **kwargs):
        super().__init__()
        if input_layout not in ("BSH", "BNSD", "TH"):
            raise ValueError(f"input_layout must be BSH, BNSD or TH, got {input_layout!r}")
        if sparse_mode not in (0, 1, 2, 3, 4):
            raise ValueError(f"sparse_mode {sparse_mode} is not supported (0-4 are)")
        self.head_num, self.keep_prob, self.scale = head_num, float(keep_prob), float(scale_value)
        self.pre_tokens, self.next_tokens = int(pre_tokens), int(next_tokens)
        self.layout, self.sparse_mode = input_layout, sparse_mode
        self.use_attention_mask, self.use_alibi_mask = use_attention_mask, use_alibi_mask
        self.use_actual_seqlen = use_actual_seqlen

    def _split(self, x: torch.Tensor, heads: Optional[int] = None):
        """→ ``[B, S, heads, D]``."""
        if self.layout == "BNSD":
            return x.transpose(1, 2)
        B, S, H = x.shape
        if heads is None:
            heads = self.head_num
        return x.view(B, S, heads, H // heads)

    def _merge(self, o: torch.Tensor):
        if self.layout == "BNSD":
            return o.transpose(1, 2)
        return o.reshape(o.shape[0], o.shape[1], -1)

    def _structural_mask(self, Sq: int, Sk: int, device):
        """True = discard, from ``sparse_mode`` / ``pre_tokens`` / ``next_tokens``; None when nothing is masked."""
        qi = torch.arange(Sq, device=device)[:, None]
        ki = torch.arange(Sk, device=device)[None, :]
        if self.sparse_mode == 2:
            return ki > qi
        if self.sparse_mode == 3:
            return ki > qi + (Sk - Sq)
        if self.sparse_mode == 4 or self.pre_tokens < _INT_MAX or self.next_tokens < _INT_MAX:
            off = Sk - Sq if self.sparse_mode == 4 else 0
            return (ki > qi + off + self.next_tokens) | (ki < qi + off - self.pre_tokens)
        return None

    def forward(self, query, key, value, attn_mask=None, alibi_mask=None, padding_mask=None, prefix=None,
                actual_seq_qlen=None, actual_seq_kvlen=None):
        if padding_mask is not None or prefix is not None:
            raise NotImplementedError("padding_mask and prefix are reserved arguments without an implementation")
        if self.layout == "TH":
            return self._packed(query, key, value, actual_seq_qlen, actual_seq_kvlen)
        D = (query.shape[-1] // self.head_num) if self.layout == "BSH" else query.shape[-1]
        q = self._split(query)
        k = self._split(key, key.shape[-1] // D if self.layout == "BSH" else None)
        v = self._split(value, value.shape[-1] // D if self.layout == "BSH" else None)
        Sq, Sk = q.shape[1], k.shape[1]
        dropout = self.keep_prob < 1.0 and self.training
        plain_causal = (self.sparse_mode in (2, 3) and Sq == Sk and alibi_mask is None and not dropout
                        and (attn_mask is None or not self.use_attention_mask or self.sparse_mode in (2, 3)))
        if plain_causal:
            return self._merge(Fn.attention(q.contiguous(), k.contiguous(), v.contiguous(), causal=True, scale=self.scale))
        discard = self._structural_mask(Sq, Sk, q.device) if (attn_mask is None or self.sparse_mode in (2, 3, 4)) else None
        if attn_mask is not None and self.sparse_mode in (0, 1):
            m = attn_mask.to(torch.bool)
            while m.dim() < 4:
                m = m.unsqueeze(0)
            discard = m if discard is None else (discard | m)
        rep = q.shape[2] // k.shape[2]
        qf = q.float().permute(0, 2, 1, 3)
        kf = k.float().permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
        vf = v.float().permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
        s = qf @ kf.transpose(-1, -2) * self.scale
        if alibi_mask is not None:
            s = s + alibi_mask.float()
        if discard is not None:
            s = s.masked_fill(discard, float("-inf"))
        p = torch.nan_to_num(torch.softmax(s, dim=-1))
        if dropout:
            p = torch.nn.functional.dropout(p, 1.0 - self.keep_prob)
        return self._merge((p @ vf).permute(0, 2, 1, 3).to(query.dtype))

    def _packed(self, query, key, value, actual_seq_qlen, actual_seq_kvlen):
        """Packed tokens: documents end at the cumulative ``actual_seq_qlen``; attention is causal inside a document."""
        if actual_seq_qlen is None:
            raise ValueError("the TH layout needs actual_seq_qlen (cumulative document ends)")
        ends = [int(e) for e in (actual_seq_qlen.tolist() if isinstance(actual_seq_qlen, torch.Tensor) else actual_seq_qlen)]
        D = query.shape[-1] // self.head_num
        out, start = [], 0
        for end in ends:
            if end <= start:
                continue
            q = query[start:end].view(1, end - start, self.head_num, D)
            k = key[start:end].view(1, end - start, -1, D)
            v = value[start:end].view(1, end - start, -1, D)
            out.append(Fn.attention(q.contiguous(), k.contiguous(), v.contiguous(), causal=True, scale=self.scale)
                       .reshape(end - start, -1))
            start = end
        return torch.cat(out, dim=0).to(query.dtype)
