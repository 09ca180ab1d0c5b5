"""Front-end of the hand-written flash-attention kernels (``csrc/flash_attention.cu``).

``flash_attention_packed`` is the training entry: it takes the packed ``[T, nq + 2·nkv, 128]`` buffer that
the QKV projection (and the in-place RoPE kernel) produced and returns ``[T, nq·128]``; its backward
writes one packed gradient buffer, so no concatenation or copy sits between attention and the QKV GEMM.
"""
from __future__ import annotations

import math

import torch

from . import _lib

HEAD_DIM = 128
TILE = 128


def _ok(seq: int, hd: int, nq: int, nkv: int, dtype) -> bool:
    return dtype == torch.bfloat16 and hd == HEAD_DIM and seq % TILE == 0 and nq % nkv == 0


def supported(q, k, v, causal) -> bool:
    """True when the native kernel covers this problem (bf16, head dim 128, equal q/k lengths)."""
    return (q.is_cuda and v.shape[-1] == HEAD_DIM and q.shape[1] == k.shape[1]
            and _ok(q.shape[1], q.shape[-1], q.shape[2], k.shape[2], q.dtype)
            and q.stride(-1) == 1 and k.stride(-1) == 1 and v.stride(-1) == 1)


def _scratch(device, nbytes: int) -> torch.Tensor:
    from .functional import _scratch as _f32
    return _f32(device, (nbytes + 3) // 4)


def document_tables(cu_seqlens: torch.Tensor = None, actual_seq_len: torch.Tensor = None, B: int = 1, S: int = 0):
    """``(doc_start, doc_end)`` int32 ``[B, S]`` tables the packed-sequence kernels take: for every token the first
    position of its document inside its row and one past the last. From ``cu_seqlens`` (``[n + 1]`` boundaries of one
    packed row, ``B`` must be 1) or from ``actual_seq_len`` (``[B, P]`` cumulative document ends per row, padded with
    ``S``, as the datasets emit them with ``create_compressed_eod_mask``)."""
    if cu_seqlens is not None:
        ends = cu_seqlens[1:].reshape(1, -1).to(torch.int64)
    else:
        ends = actual_seq_len.reshape(B, -1).to(torch.int64)
    dev = ends.device
    ends, _ = torch.sort(torch.clamp(ends, max=S), dim=1)
    pos = torch.arange(S, device=dev, dtype=torch.int64).unsqueeze(0).expand(ends.shape[0], S).contiguous()
    idx = torch.searchsorted(ends, pos, right=True)                      # first end > position
    padded = torch.cat([ends, torch.full((ends.shape[0], 1), S, dtype=torch.int64, device=dev)], dim=1)
    doc_end = padded.gather(1, idx)
    starts = torch.cat([torch.zeros((ends.shape[0], 1), dtype=torch.int64, device=dev), ends], dim=1)
    doc_start = starts.gather(1, idx)
    return doc_start.to(torch.int32).contiguous(), doc_end.to(torch.int32).contiguous()


def _fwd(q, k, v, B, S, nq, nkv, q_ld, k_ld, v_ld, causal, scale, need_lse=True, doc_start=None):
    T = B * S
    out = torch.empty((T, nq * HEAD_DIM), dtype=torch.bfloat16, device=q.device)
    lse = torch.empty((B, nq, S), dtype=torch.float32, device=q.device) if need_lse else None
    st = _lib.status_word(q.device)
    if doc_start is not None:
        rc = _lib.get_lib().mfb_flash_attn_fwd2_varlen(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                                                       _lib.ptr(lse), doc_start.data_ptr(), B, S, S, nq, nkv, q_ld, k_ld,
                                                       v_ld, out.stride(0), int(causal), 0, float(scale), st.data_ptr(),
                                                       _lib.stream_ptr())
        _lib.check(rc, "mfb_flash_attn_fwd2_varlen")
        _lib.count_launch()
        return out, lse
    rc = _lib.get_lib().mfb_flash_attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), _lib.ptr(lse),
                                           B, S, S, nq, nkv, q_ld, k_ld, v_ld, out.stride(0), int(causal),
                                           float(scale), st.data_ptr(), _lib.stream_ptr())
    _lib.check(rc, "mfb_flash_attn_fwd")
    _lib.count_launch()
    return out, lse


class _PackedAttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, packed, B, S, nq, nkv, causal, scale, doc_start=None, doc_end=None):
        # packed: [T, nq + 2 nkv, 128] contiguous
        W = packed.shape[1] * HEAD_DIM
        q = packed
        k = packed[:, nq:]
        v = packed[:, nq + nkv:]
        from ..parallel.recompute import cached_output
        out, lse = cached_output(lambda: _fwd(q, k, v, B, S, nq, nkv, W, W, W, causal, scale, doc_start=doc_start))
        ctx.save_for_backward(packed, out, lse)
        ctx.meta = (B, S, nq, nkv, causal, scale)
        ctx.docs = (doc_start, doc_end)
        return out

    @staticmethod
    def backward(ctx, dout):
        packed, out, lse = ctx.saved_tensors
        B, S, nq, nkv, causal, scale = ctx.meta
        W = packed.shape[1] * HEAD_DIM
        dout = dout.contiguous()
        dpacked = torch.empty_like(packed)
        lib = _lib.get_lib()
        scratch = _scratch(packed.device, lib.mfb_flash_attn_bwd_scratch_bytes_ex(B, S, S, nq, nkv))
        st = _lib.status_word(packed.device)
        k, v = packed[:, nq:], packed[:, nq + nkv:]
        dk, dv = dpacked[:, nq:], dpacked[:, nq + nkv:]
        doc_start, doc_end = ctx.docs
        if doc_start is not None:
            rc = lib.mfb_flash_attn_bwd2_varlen(packed.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), dout.data_ptr(),
                                                lse.data_ptr(), doc_start.data_ptr(), doc_end.data_ptr(), dpacked.data_ptr(),
                                                dk.data_ptr(), dv.data_ptr(), scratch.data_ptr(), B, S, S, nq, nkv, W, W, W,
                                                out.stride(0), dout.stride(0), W, W, W, int(causal), 0, float(scale),
                                                st.data_ptr(), _lib.stream_ptr())
            _lib.check(rc, "mfb_flash_attn_bwd2_varlen")
            _lib.count_launch(4)
            return dpacked, None, None, None, None, None, None, None, None
        rc = lib.mfb_flash_attn_bwd(packed.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), dout.data_ptr(),
                                    lse.data_ptr(), dpacked.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                                    scratch.data_ptr(), B, S, nq, nkv, W, W, W, out.stride(0), dout.stride(0), W, W, W,
                                    int(causal), float(scale), st.data_ptr(), _lib.stream_ptr())
        _lib.check(rc, "mfb_flash_attn_bwd")
        _lib.count_launch(4)
        return dpacked, None, None, None, None, None, None, None, None


def packed_supported(packed: torch.Tensor, S: int, nq: int, nkv: int) -> bool:
    return (packed.is_cuda and packed.is_contiguous() and packed.dim() == 3
            and _ok(S, packed.shape[-1], nq, nkv, packed.dtype))


def flash_attention_packed(packed: torch.Tensor, B: int, S: int, nq: int, nkv: int, causal: bool = True,
                           scale: float = None, doc_start: torch.Tensor = None, doc_end: torch.Tensor = None) -> torch.Tensor:
    """Attention over a packed qkv buffer ``[B·S, nq + 2·nkv, 128]`` → ``[B·S, nq·128]``. With ``doc_start`` /
    ``doc_end`` (``document_tables``) every row holds several documents and a token attends inside its own only."""
    scale = scale if scale is not None else 1.0 / math.sqrt(HEAD_DIM)
    return _PackedAttnFn.apply(packed, B, S, nq, nkv, causal, scale, doc_start, doc_end)


class _AttnFn(torch.autograd.Function):
    """Separate q/k/v tensors ``[B, S, h, 128]`` (any row pitch); used by inference prefill and the ring steps."""

    @staticmethod
    def forward(ctx, q, k, v, causal, scale):
        B, S, nq, _ = q.shape
        nkv = k.shape[2]
        from ..parallel.recompute import cached_output
        out, lse = cached_output(lambda: _fwd(q, k, v, B, S, nq, nkv, q.stride(1), k.stride(1), v.stride(1), causal, scale))
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.meta = (causal, scale)
        return out.view(B, S, nq, HEAD_DIM)

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse = ctx.saved_tensors
        causal, scale = ctx.meta
        B, S, nq, _ = q.shape
        nkv = k.shape[2]
        dout = dout.contiguous()
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        if not (dq.is_contiguous() and dk.is_contiguous() and dv.is_contiguous()):
            dq = torch.empty(q.shape, dtype=q.dtype, device=q.device)
            dk = torch.empty(k.shape, dtype=k.dtype, device=k.device)
            dv = torch.empty(v.shape, dtype=v.dtype, device=v.device)
        lib = _lib.get_lib()
        scratch = _scratch(q.device, lib.mfb_flash_attn_bwd_scratch_bytes_ex(B, S, S, nq, nkv))
        st = _lib.status_word(q.device)
        rc = lib.mfb_flash_attn_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), dout.data_ptr(),
                                    lse.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), scratch.data_ptr(),
                                    B, S, nq, nkv, q.stride(1), k.stride(1), v.stride(1), out.stride(0),
                                    nq * HEAD_DIM, dq.stride(1), dk.stride(1), dv.stride(1), int(causal), float(scale),
                                    st.data_ptr(), _lib.stream_ptr())
        _lib.check(rc, "mfb_flash_attn_bwd")
        _lib.count_launch(4)
        return dq, dk, dv, None, None


def flash_attention(q, k, v, causal=True, scale=None):
    """q: ``[B, S, Hq, 128]``, k/v: ``[B, S, Hkv, 128]`` (views with unit inner stride and the batch and
    sequence axes mergeable into one row axis) → ``[B, S, Hq, 128]``."""
    scale = scale if scale is not None else 1.0 / math.sqrt(HEAD_DIM)
    for t in (q, k, v):
        if t.stride(0) != t.shape[1] * t.stride(1) or t.stride(2) != HEAD_DIM:
            return _AttnFn.apply(q.contiguous(), k.contiguous(), v.contiguous(), causal, scale)
    return _AttnFn.apply(q, k, v, causal, scale)


def mla_supported(q, k, v) -> bool:
    """Forward-only kernel for the multi-latent-attention shape: q/k heads of 192, v heads of 128, bf16, sequence a
    multiple of 128, the same number of q and k heads."""
    return (q.is_cuda and q.dtype == torch.bfloat16 and q.shape[-1] == 192 and k.shape[-1] == 192
            and v.shape[-1] == HEAD_DIM and q.shape[1] % TILE == 0 and q.shape[1] == k.shape[1]
            and q.shape[2] % k.shape[2] == 0 and k.shape[2] == v.shape[2])


def mla_forward(q, k, v, causal: bool = True, scale=None):
    """q, k ``[B, S, h, 192]``, v ``[B, S, h, 128]`` → ``[B, S, h, 128]``. Inference only (no backward kernel for this
    shape: training takes the autograd path of ``functional.attention``)."""
    B, S, nq, dq = q.shape
    nkv = k.shape[2]
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    scale = scale if scale is not None else 1.0 / math.sqrt(dq)
    out = torch.empty((B * S, nq * HEAD_DIM), dtype=torch.bfloat16, device=q.device)
    st = _lib.status_word(q.device)
    rc = _lib.get_lib().mfb_flash_attn_fwd_mla(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), None, B, S, S,
                                               nq, nkv, nq * dq, nkv * dq, nkv * HEAD_DIM, out.stride(0), int(causal), 0,
                                               float(scale), st.data_ptr(), _lib.stream_ptr())
    _lib.check(rc, "mfb_flash_attn_fwd_mla")
    _lib.count_launch()
    return out.view(B, S, nq, HEAD_DIM)


# ---- rectangular causal attention: Sq queries at key positions [q_offset, q_offset + Sq) of Sk keys ------------
def rect_forward(q, k, v, q_offset: int, causal: bool, scale: float):
    """Raw forward: q ``[B,Sq,Hq,128]``, k/v ``[B,Sk,Hkv,128]`` contiguous → ``(out [B*Sq, Hq*128], lse [B,Hq,Sq])``."""
    B, Sq, nq, _ = q.shape
    Sk, nkv = k.shape[1], k.shape[2]
    out = torch.empty((B * Sq, nq * HEAD_DIM), dtype=torch.bfloat16, device=q.device)
    lse = torch.empty((B, nq, Sq), dtype=torch.float32, device=q.device)
    st = _lib.status_word(q.device)
    rc = _lib.get_lib().mfb_flash_attn_fwd_ex(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(),
                                              B, Sq, Sk, nq, nkv, q.stride(1), k.stride(1), v.stride(1), out.stride(0),
                                              int(causal), int(q_offset), float(scale), st.data_ptr(), _lib.stream_ptr())
    _lib.check(rc, "mfb_flash_attn_fwd_ex")
    _lib.count_launch()
    return out, lse


def rect_backward(q, k, v, out, lse, dout, dk, dv, q_offset: int, causal: bool, scale: float):
    """Raw backward: returns ``dq``; writes ``dk`` / ``dv`` (``[B,Sk,Hkv,128]``, every key row, zeros where no query looks)."""
    B, Sq, nq, _ = q.shape
    Sk, nkv = k.shape[1], k.shape[2]
    dq = torch.empty(q.shape, dtype=q.dtype, device=q.device)
    lib = _lib.get_lib()
    scratch = _scratch(q.device, lib.mfb_flash_attn_bwd_scratch_bytes_ex(B, Sq, Sk, nq, nkv))
    st = _lib.status_word(q.device)
    rc = lib.mfb_flash_attn_bwd_ex(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), dout.data_ptr(), lse.data_ptr(),
                                   dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), scratch.data_ptr(), B, Sq, Sk, nq, nkv,
                                   q.stride(1), k.stride(1), v.stride(1), out.stride(0), nq * HEAD_DIM, dq.stride(1),
                                   dk.stride(1), dv.stride(1), int(causal), int(q_offset), float(scale), st.data_ptr(),
                                   _lib.stream_ptr())
    _lib.check(rc, "mfb_flash_attn_bwd_ex")
    _lib.count_launch(4)
    return dq


class _RectAttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, q_offset, causal, scale):
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        out, lse = rect_forward(q, k, v, q_offset, causal, scale)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.meta = (q_offset, causal, scale)
        B, Sq, nq, _ = q.shape
        return out.view(B, Sq, nq, HEAD_DIM)

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse = ctx.saved_tensors
        q_offset, causal, scale = ctx.meta
        dk, dv = torch.empty_like(k), torch.empty_like(v)
        dq = rect_backward(q, k, v, out, lse, dout.contiguous(), dk, dv, q_offset, causal, scale)
        return dq, dk, dv, None, None, None


def rect_supported(q, k, v) -> bool:
    return (q.is_cuda and q.dtype == torch.bfloat16 and q.shape[-1] == HEAD_DIM and v.shape[-1] == HEAD_DIM
            and q.shape[1] % TILE == 0 and k.shape[1] % TILE == 0 and q.shape[2] % k.shape[2] == 0)


def flash_attention_rect(q, k, v, q_offset: int = 0, causal: bool = True, scale=None):
    """Attention of ``Sq`` queries over ``Sk`` keys, query ``i`` sitting at key position ``q_offset + i``
    (``q_offset`` a multiple of 128): prefix / chunked-prefill / context-parallel shapes."""
    scale = scale if scale is not None else 1.0 / math.sqrt(HEAD_DIM)
    return _RectAttnFn.apply(q, k, v, int(q_offset), bool(causal), float(scale))
