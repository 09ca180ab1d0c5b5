"""Differentiable front-ends of the sm_100a kernels.

Each op has two bodies: the CUDA kernel from ``libmfb200.so`` (taken whenever the tensors live on a
GPU; a missing library raises) and a plain PyTorch body that serves CPU runs and is the numerical
oracle of the kernel tests. The GEMM additionally has a ``"cublas"`` backend (``torch.matmul``),
which is the library baseline the hand-written tcgen05 kernel is measured against.
"""
from __future__ import annotations

import math
import os
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from . import _lib

_GEMM_BACKEND = "tcgen05"
_ATTN_BACKEND = "auto"


def set_gemm_backend(name: str):
    """``"tcgen05"`` (hand-written kernel, default) or ``"cublas"`` (torch.matmul baseline)."""
    global _GEMM_BACKEND
    if name not in ("tcgen05", "cublas"):
        raise ValueError(f"unknown GEMM backend {name!r}")
    _GEMM_BACKEND = name


def get_gemm_backend() -> str:
    return _GEMM_BACKEND


def set_attention_backend(name: str):
    """``"auto"``/``"native"`` (hand-written kernel on CUDA) or ``"sdpa"`` (library baseline)."""
    global _ATTN_BACKEND
    if name not in ("auto", "native", "sdpa"):
        raise ValueError(f"unknown attention backend {name!r}")
    _ATTN_BACKEND = name


def get_attention_backend() -> str:
    return _ATTN_BACKEND


class _NoGradCtx:
    """Stand-in for the autograd context of a ``torch.autograd.Function`` when gradients are off: the forward
    implementation then runs as a plain call (``Function.apply`` costs tens of microseconds of host time per call,
    which is what bounds a decode step made of small kernels)."""
    needs_input_grad = ()
    saved_tensors = ()

    def save_for_backward(self, *tensors):
        pass

    def mark_non_differentiable(self, *tensors):
        pass

    def mark_dirty(self, *tensors):
        pass

    def set_materialize_grads(self, value):
        pass


def apply_fn(fn, *args):
    """``fn.apply(*args)`` with gradients enabled, ``fn.forward`` on a throw-away context otherwise."""
    if torch.is_grad_enabled():
        return fn.apply(*args)
    return fn.forward(_NoGradCtx(), *args)



def _cached_output(compute):
    from ..parallel.recompute import cached_output
    return cached_output(compute)


def _on_gpu(t: torch.Tensor) -> bool:
    return t.is_cuda


def _aligned(t: torch.Tensor) -> bool:
    return t.data_ptr() % 16 == 0 and (t.stride(0) * t.element_size()) % 16 == 0 and t.stride(-1) == 1


# =================================================================================================
# GEMM
# =================================================================================================
_OUT_MODES = {(torch.bfloat16, False): 0, (torch.float32, False): 1, (torch.float32, True): 2,
              (torch.bfloat16, True): 3}


def _decode_gemm_ok(M: int, K: int, a: torch.Tensor, b: torch.Tensor) -> bool:
    return _DECODE_GEMM and M <= 64 and K >= 64 and K % 8 == 0 and a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16


def decode_linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """``x W^T + bias`` for 1 - 64 rows of ``x`` on the weight-on-rows kernel with the bias added in its epilogue; None
    when the kernel does not serve the call (the caller then takes the general path)."""
    if not (_on_gpu(x) and _GEMM_BACKEND == "tcgen05" and x.dim() == 2 and w.dim() == 2 and _decode_gemm_ok(x.shape[0], x.shape[1], x, w)):
        return None
    if bias is not None and (bias.dtype != torch.bfloat16 or not bias.is_contiguous() or bias.numel() != w.shape[0]):
        return None
    if not _aligned(x):
        x = x.contiguous()
    if not _aligned(w):
        w = w.contiguous()
    out = torch.empty((x.shape[0], w.shape[0]), dtype=torch.bfloat16, device=x.device)
    rc = _lib.get_lib().mfb_gemm_bf16_decode(x.data_ptr(), w.data_ptr(), out.data_ptr(), _lib.ptr(bias), x.shape[0], w.shape[0],
                                             x.shape[1], x.stride(0), w.stride(0), out.stride(0), _DECODE_GEMM_KS,
                                             _lib.status_word(x.device).data_ptr(), _lib.stream_ptr())
    _lib.check(rc, "mfb_gemm_bf16_decode")
    _lib.count_launch()
    return out


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
         out: Optional[torch.Tensor] = None, out_dtype: torch.dtype = torch.bfloat16,
         accumulate: bool = False, sm_limit: int = 0) -> torch.Tensor:
    """``D[M,N] = sum_k A(m,k) B(n,k)`` with fp32 accumulation.

    ``a`` is ``[M,K]`` (or ``[K,M]`` when ``a_mn``), ``b`` is ``[N,K]`` (or ``[K,N]`` when ``b_mn``).
    ``accumulate`` adds into ``out`` (TMA reduce-add) instead of overwriting it.
    """
    M = a.shape[1] if a_mn else a.shape[0]
    K = a.shape[0] if a_mn else a.shape[1]
    N = b.shape[1] if b_mn else b.shape[0]
    Kb = b.shape[0] if b_mn else b.shape[1]
    if K != Kb:
        raise ValueError(f"gemm: reduction extents differ ({K} vs {Kb})")
    if out is not None:
        out_dtype = out.dtype
    use_kernel = _on_gpu(a) and _GEMM_BACKEND == "tcgen05" and a.dtype == torch.bfloat16
    if not use_kernel:
        am = a.t() if a_mn else a
        bm = b if b_mn else b.t()
        if a.is_cuda:
            res = torch.matmul(am, bm)
        else:
            res = torch.matmul(am.float(), bm.float())
        if out is None:
            return res.to(out_dtype)
        if accumulate:
            out.add_(res.to(out.dtype))
        else:
            out.copy_(res)
        return out
    if not _aligned(a):
        a = a.contiguous()
    if not _aligned(b):
        b = b.contiguous()
    if out is None:
        if accumulate:
            raise ValueError("gemm: accumulate needs an output tensor")
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    elif not _aligned(out) or out.shape != (M, N):
        raise ValueError("gemm: output must be a 16-byte aligned [M,N] tensor with unit inner stride")
    mode = _OUT_MODES[(out.dtype, bool(accumulate))]
    lib = _lib.get_lib()
    st = _lib.status_word(a.device)
    if _DECODE_GEMM and M <= 64 and mode == 0 and not a_mn and not b_mn and K >= 64 and K % 8 == 0 \
            and b.dtype == torch.bfloat16:
        # a few rows of activations: the weight rows go on the MMA rows and every weight is streamed once
        rc = lib.mfb_gemm_bf16_decode(a.data_ptr(), b.data_ptr(), out.data_ptr(), None, M, N, K, a.stride(0), b.stride(0),
                                      out.stride(0), _DECODE_GEMM_KS, st.data_ptr(), _lib.stream_ptr())
        _lib.check(rc, "mfb_gemm_bf16_decode")
        _lib.count_launch()
        return out
    if _PAIR_GEMM and M >= 256 and N >= 256 and K >= 64:
        # 256 x 256 tiles on CTA pairs; the tail wave is split along K through a per-stream workspace
        ws = _pair_workspace(a.device) if _PAIR_SLICES > 1 and mode < 2 else None
        rc = lib.mfb_gemm_bf16_pair(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), b.stride(0),
                                    out.stride(0), int(a_mn), int(b_mn), mode, _lib.ptr(ws), _PAIR_SLICES,
                                    st.data_ptr(), int(sm_limit), _lib.stream_ptr())
        _lib.check(rc, "mfb_gemm_bf16_pair")
        _lib.count_launch()
        return out
    rc = lib.mfb_gemm_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), b.stride(0),
                           out.stride(0), int(a_mn), int(b_mn), mode, 0, 1, 0, 0, 0, 0, st.data_ptr(),
                           int(sm_limit), _lib.stream_ptr())
    _lib.check(rc, "mfb_gemm_bf16")
    _lib.count_launch()
    return out


# Dense GEMMs of at least one 256 x 256 tile run on CTA pairs (``gemm_tcgen05_2cta.cu``); ``MFB_GEMM_PAIR=0``
# keeps the single-CTA kernel for A/B measurements, ``MFB_GEMM_PAIR_SLICES`` bounds the K split of the tail wave.
_PAIR_GEMM = os.environ.get("MFB_GEMM_PAIR", "1") != "0"
# Products with at most 64 rows of activations (decode steps) take ``gemm_bf16_decode.cu``; ``MFB_BF16_DECODE_KERNEL=0``
# keeps the general kernels, ``MFB_BF16_DECODE_KS`` fixes its K split (1, 2, 4, 8; 16 = two CTAs per SM) for measurements.
_DECODE_GEMM = os.environ.get("MFB_BF16_DECODE_KERNEL", "1") != "0"
_DECODE_GEMM_KS = int(os.environ.get("MFB_BF16_DECODE_KS", "0"))


def set_decode_gemm(enabled: bool, force_ks: int = 0):
    """Switch the small-row-count GEMM kernel (and fix its K split) at run time."""
    global _DECODE_GEMM, _DECODE_GEMM_KS
    _DECODE_GEMM, _DECODE_GEMM_KS = bool(enabled), int(force_ks)

_PAIR_SLICES = int(os.environ.get("MFB_GEMM_PAIR_SLICES", "4"))
_pair_ws_cache: dict = {}


def set_pair_gemm(enabled: bool, max_slices: Optional[int] = None):
    """Switch the CTA-pair GEMM (and the K split of its tail wave) at run time."""
    global _PAIR_GEMM, _PAIR_SLICES
    _PAIR_GEMM = bool(enabled)
    if max_slices is not None:
        _PAIR_SLICES = int(max_slices)


def _pair_workspace(device) -> torch.Tensor:
    """Zero-initialised workspace of the split tail wave, one per (device, stream): two GEMMs that overlap on
    the GPU must not share partial tiles or flags."""
    key = (torch.device(device).index or 0, _lib.stream_ptr())
    t = _pair_ws_cache.get(key)
    if t is None:
        nbytes = int(_lib.get_lib().mfb_gemm_pair_workspace_bytes())
        t = torch.zeros(nbytes, dtype=torch.uint8, device=device)
        _pair_ws_cache[key] = t
    return t


def grouped_gemm(a: torch.Tensor, b: torch.Tensor, block_group: torch.Tensor, num_blocks: torch.Tensor,
                 *, b_mn: bool = False, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Ragged-M grouped GEMM for MoE experts.

    ``a``: ``[R, K]`` rows sorted by expert, every expert segment padded to a multiple of 128 rows.
    ``b``: ``[G, N, K]`` (or ``[G, K, N]`` when ``b_mn``). ``block_group[i]`` = expert of the i-th
    128-row block; ``num_blocks`` = device scalar with the number of blocks in use.
    """
    G = b.shape[0]
    R, K = a.shape
    N = b.shape[2] if b_mn else b.shape[1]
    if out is None:
        out = torch.empty((R, N), dtype=a.dtype, device=a.device)
    if not (_on_gpu(a) and _GEMM_BACKEND == "tcgen05" and a.dtype == torch.bfloat16):
        nb = int(num_blocks.item())
        bg = block_group[:nb].tolist()
        out.zero_()
        for i, g in enumerate(bg):
            rows = slice(i * 128, (i + 1) * 128)
            w = b[g].float() if b_mn else b[g].float().t()
            out[rows] = (a[rows].float() @ w).to(out.dtype)
        return out
    lib = _lib.get_lib()
    st = _lib.status_word(a.device)
    b2 = b.reshape(-1, b.shape[-1])
    rc = lib.mfb_gemm_bf16(a.data_ptr(), b2.data_ptr(), out.data_ptr(), R, N, K, a.stride(0), b2.stride(0),
                           out.stride(0), 0, int(b_mn), 0, 1, G, block_group.data_ptr(),
                           num_blocks.data_ptr(), 0, R, st.data_ptr(), 0, _lib.stream_ptr())
    _lib.check(rc, "mfb_gemm_bf16[grouped]")
    _lib.count_launch()
    return out


def grouped_wgrad(dy: torch.Tensor, x: torch.Tensor, group_offsets: torch.Tensor, num_groups: int,
                  out: torch.Tensor, accumulate: bool = False) -> torch.Tensor:
    """Per-expert weight gradient ``out[g] (+)= dy[rows_g]^T x[rows_g]`` with ``out`` = ``[G, N_out, K_in]``."""
    R, Nout = dy.shape
    Kin = x.shape[1]
    if not (_on_gpu(dy) and _GEMM_BACKEND == "tcgen05" and dy.dtype == torch.bfloat16):
        offs = group_offsets.tolist()
        for g in range(num_groups):
            rows = slice(offs[g], offs[g + 1])
            val = dy[rows].float().t() @ x[rows].float()
            if accumulate:
                out[g] += val.to(out.dtype)
            else:
                out[g] = val.to(out.dtype)
        return out
    lib = _lib.get_lib()
    st = _lib.status_word(dy.device)
    o2 = out.reshape(-1, Kin)
    mode = _OUT_MODES[(out.dtype, bool(accumulate))]
    rc = lib.mfb_gemm_bf16(dy.data_ptr(), x.data_ptr(), o2.data_ptr(), Nout, Kin, 0, dy.stride(0), x.stride(0),
                           o2.stride(0), 1, 1, mode, 2, num_groups, 0, 0, group_offsets.data_ptr(), R,
                           st.data_ptr(), 0, _lib.stream_ptr())
    _lib.check(rc, "mfb_gemm_bf16[grouped wgrad]")
    _lib.count_launch()
    return out


class _LinearFn(torch.autograd.Function):
    """``y = x W^T``; weight gradient goes to ``W.main_grad`` (accumulating) when that buffer exists."""

    @staticmethod
    def forward(ctx, x, w):
        ctx.save_for_backward(x, w)
        x2 = x.reshape(-1, x.shape[-1])
        y = _cached_output(lambda: gemm(x2, w, out_dtype=x.dtype))   # a selective-recompute region runs the product once only
        if x.dim() == 2:
            return y  # not a view: later in-place kernels (RoPE) may write into it
        return y.reshape(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        x2 = x.reshape(-1, x.shape[-1])
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, w, b_mn=True, out_dtype=x.dtype).reshape(x.shape)
        if ctx.needs_input_grad[1]:
            main_grad = getattr(w, "main_grad", None)
            if main_grad is not None:
                gemm(dy2, x2, a_mn=True, b_mn=True, out=main_grad, accumulate=True)
                dw = None
            else:
                dw = gemm(dy2, x2, a_mn=True, b_mn=True, out_dtype=w.dtype)
        return dx, dw


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    from ..parallel.recompute import current_cache
    if current_cache() is not None and torch.is_grad_enabled():
        # inside a selective-recompute region every product goes through the function that knows the output cache
        y = _LinearFn.apply(x, w)
        return y if bias is None else y + bias
    if not _on_gpu(x) or x.dtype != torch.bfloat16 or _GEMM_BACKEND != "tcgen05":
        if getattr(w, "main_grad", None) is not None and x.is_cuda:
            y = apply_fn(_LinearFn, x, w)
            return y if bias is None else y + bias
        return F.linear(x, w, bias)
    if bias is not None and not (torch.is_grad_enabled() and (x.requires_grad or w.requires_grad or bias.requires_grad)):
        x2 = x.reshape(-1, x.shape[-1])
        y = decode_linear(x2, w, bias) if x2.shape[0] <= 64 else None      # decode step: bias added by the GEMM's epilogue
        if y is not None:
            return y if x.dim() == 2 else y.reshape(*x.shape[:-1], w.shape[0])
    y = apply_fn(_LinearFn, x, w)
    if bias is not None:
        y = y + bias
    return y


# =================================================================================================
# RMSNorm (+ fused residual add)
# =================================================================================================
def rmsnorm_reference(x, w, eps, residual=None):
    h = x if residual is None else (x + residual)
    hf = h.float()
    rstd = torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + eps)
    y = (hf * rstd * w.float()).to(x.dtype)
    return y, h


_scratch_cache: dict = {}


def _scratch(device, nfloats: int) -> torch.Tensor:
    """Reusable fp32 scratch of at least ``nfloats`` elements for the CURRENT stream of ``device``. The cache is keyed
    by (device, stream): kernels of two streams (``MicroBatchInterleaved`` copies, side-stream reductions) may be in
    flight together and must not share partial sums. A buffer is allocated while its stream is current, so the caching
    allocator ties the block to that stream; when a request outgrows the buffer the old one is dropped, which is safe
    because every user of it was queued on the same stream before the new allocation."""
    key = (torch.device(device).index or 0, _lib.stream_ptr())
    t = _scratch_cache.get(key)
    if t is None or t.numel() < nfloats:
        t = torch.empty(max(nfloats, 1 << 20), dtype=torch.float32, device=device)
        _scratch_cache[key] = t
    return t


class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, residual, w, eps):
        shape = x.shape
        H = shape[-1]
        x2 = x.reshape(-1, H)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        T = x2.shape[0]
        y = torch.empty_like(x2)
        rstd = torch.empty(T, dtype=torch.float32, device=x.device)
        lib = _lib.get_lib()
        if residual is not None:
            r2 = residual.reshape(-1, H)
            if not r2.is_contiguous():
                r2 = r2.contiguous()
            h = torch.empty_like(x2)
            rc = lib.mfb_rmsnorm_fwd(x2.data_ptr(), r2.data_ptr(), w.data_ptr(), y.data_ptr(), h.data_ptr(),
                                     rstd.data_ptr(), T, H, float(eps), _lib.stream_ptr())
        else:
            h = x2
            rc = lib.mfb_rmsnorm_fwd(x2.data_ptr(), 0, w.data_ptr(), y.data_ptr(), 0, rstd.data_ptr(), T, H,
                                     float(eps), _lib.stream_ptr())
        _lib.check(rc, "mfb_rmsnorm_fwd")
        _lib.count_launch()
        ctx.save_for_backward(h, w, rstd)
        ctx.has_res = residual is not None
        ctx.shape = shape
        return y.reshape(shape), h.reshape(shape)

    @staticmethod
    def backward(ctx, dy, dh):
        h, w, rstd = ctx.saved_tensors
        T, H = h.shape
        dy2 = dy.reshape(T, H)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dres = None
        if dh is not None:
            dres = dh.reshape(T, H)
            if not dres.is_contiguous():
                dres = dres.contiguous()
        dx = torch.empty_like(h)
        lib = _lib.get_lib()
        parts = lib.mfb_rmsnorm_bwd_parts(T)
        scratch = _scratch(h.device, parts * H)
        main_grad = getattr(w, "main_grad", None)
        if main_grad is not None:
            dwf, dwb, acc, dw = main_grad.data_ptr(), 0, 1, None
        else:
            dw = torch.empty(H, dtype=torch.float32, device=h.device)
            dwf, dwb, acc = dw.data_ptr(), 0, 0
        rc = lib.mfb_rmsnorm_bwd(dy2.data_ptr(), h.data_ptr(), w.data_ptr(), rstd.data_ptr(), _lib.ptr(dres),
                                 dx.data_ptr(), dwf, dwb, acc, scratch.data_ptr(), T, H, _lib.stream_ptr())
        _lib.check(rc, "mfb_rmsnorm_bwd")
        _lib.count_launch(2)
        if dw is not None:
            dw = dw.to(w.dtype)
        dx = dx.reshape(ctx.shape)
        return dx, (dx if ctx.has_res else None), dw, None


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-5,
            residual: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Returns ``(norm(x + residual) * w, x + residual)``; the second value is the new residual stream."""
    if _on_gpu(x) and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0 \
            and x.shape[-1] <= 8192:
        return apply_fn(_RMSNormFn, x, residual, w, eps)
    return rmsnorm_reference(x, w, eps, residual)


# =================================================================================================
# SwiGLU
# =================================================================================================
def swiglu_reference(x):
    g, u = x.chunk(2, dim=-1)
    return (F.silu(g.float()) * u.float()).to(x.dtype)


class _SwiGLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        F2 = x.shape[-1]
        x2 = x.reshape(-1, F2)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        out = torch.empty((x2.shape[0], F2 // 2), dtype=x.dtype, device=x.device)
        rc = _lib.get_lib().mfb_swiglu_fwd(x2.data_ptr(), out.data_ptr(), x2.shape[0], F2 // 2, _lib.stream_ptr())
        _lib.check(rc, "mfb_swiglu_fwd")
        _lib.count_launch()
        ctx.save_for_backward(x2)
        ctx.shape = x.shape
        return out.reshape(*x.shape[:-1], F2 // 2)

    @staticmethod
    def backward(ctx, dout):
        (x2,) = ctx.saved_tensors
        d2 = dout.reshape(x2.shape[0], -1)
        if not d2.is_contiguous():
            d2 = d2.contiguous()
        din = torch.empty_like(x2)
        rc = _lib.get_lib().mfb_swiglu_bwd(x2.data_ptr(), d2.data_ptr(), din.data_ptr(), x2.shape[0],
                                           x2.shape[1] // 2, _lib.stream_ptr())
        _lib.check(rc, "mfb_swiglu_bwd")
        _lib.count_launch()
        return din.reshape(ctx.shape)


def swiglu(x: torch.Tensor) -> torch.Tensor:
    """``silu(x[..., :F]) * x[..., F:]``."""
    if _on_gpu(x) and x.dtype == torch.bfloat16 and (x.shape[-1] // 2) % 8 == 0:
        return apply_fn(_SwiGLUFn, x)
    return swiglu_reference(x)


# =================================================================================================
# RoPE (applied in place to the leading heads of a packed [T, heads, hd] buffer)
# =================================================================================================
def rope_reference(x, cos, sin, positions, n_heads, rot, interleaved=False):
    """x: [T, heads_total, hd]; rotates the first n_heads heads. cos/sin: [max_pos, rot/2] fp32."""
    T = x.shape[0]
    c = cos[positions].unsqueeze(1)  # [T,1,rot/2]
    s = sin[positions].unsqueeze(1)
    xr = x[:, :n_heads, :rot].float()
    if interleaved:
        a, b = xr[..., 0::2], xr[..., 1::2]
        o = torch.stack((a * c - b * s, b * c + a * s), dim=-1).flatten(-2)
    else:
        a, b = xr[..., : rot // 2], xr[..., rot // 2:]
        o = torch.cat((a * c - b * s, b * c + a * s), dim=-1)
    out = x.clone()
    out[:, :n_heads, :rot] = o.to(x.dtype)
    return out


class _RopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin, positions, n_heads, rot, interleaved):
        # x: [T, heads_total, hd] contiguous; modified in place
        T, _, hd = x.shape
        pos32 = positions.to(torch.int32) if positions is not None else None
        rc = _lib.get_lib().mfb_rope(x.data_ptr(), cos.data_ptr(), sin.data_ptr(), _lib.ptr(pos32), T, n_heads,
                                     hd, rot, x.stride(0), int(interleaved), 0, cos.shape[0], _lib.stream_ptr())
        _lib.check(rc, "mfb_rope")
        _lib.count_launch()
        ctx.mark_dirty(x)
        ctx.save_for_backward(cos, sin, pos32 if pos32 is not None else torch.empty(0))
        ctx.meta = (n_heads, rot, interleaved, pos32 is not None)
        return x

    @staticmethod
    def backward(ctx, dx):
        cos, sin, pos32 = ctx.saved_tensors
        n_heads, rot, interleaved, has_pos = ctx.meta
        dx = dx.contiguous().clone() if not dx.is_contiguous() else dx.clone()
        T, _, hd = dx.shape
        rc = _lib.get_lib().mfb_rope(dx.data_ptr(), cos.data_ptr(), sin.data_ptr(),
                                     pos32.data_ptr() if has_pos else 0, T, n_heads, hd, rot, dx.stride(0),
                                     int(interleaved), 1, cos.shape[0], _lib.stream_ptr())
        _lib.check(rc, "mfb_rope[bwd]")
        _lib.count_launch()
        return dx, None, None, None, None, None, None


def rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, positions: torch.Tensor, n_heads: int,
         rot: int, interleaved: bool = False) -> torch.Tensor:
    """Rotate the first ``n_heads`` heads of ``x`` ``[T, heads, hd]`` (q and k of a packed qkv buffer)."""
    if _on_gpu(x) and x.dtype == torch.bfloat16 and x.is_contiguous():
        if x.requires_grad and x.is_leaf:
            x = x.clone()
        return apply_fn(_RopeFn, x, cos, sin, positions, n_heads, rot, interleaved)
    return rope_reference(x, cos, sin, positions, n_heads, rot, interleaved)


# =================================================================================================
# Embedding
# =================================================================================================
class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, table, vocab_start):
        flat = ids.reshape(-1).to(torch.int64).contiguous()
        T = flat.numel()
        H = table.shape[1]
        out = torch.empty((T, H), dtype=table.dtype, device=table.device)
        rc = _lib.get_lib().mfb_embedding_fwd(flat.data_ptr(), table.data_ptr(), out.data_ptr(), T, H,
                                              int(vocab_start), table.shape[0], _lib.stream_ptr())
        _lib.check(rc, "mfb_embedding_fwd")
        _lib.count_launch()
        ctx.save_for_backward(flat)
        ctx.table = table
        ctx.vocab_start = vocab_start
        return out.reshape(*ids.shape, H)

    @staticmethod
    def backward(ctx, dout):
        (flat,) = ctx.saved_tensors
        table = ctx.table
        H = table.shape[1]
        d2 = dout.reshape(-1, H)
        if not d2.is_contiguous():
            d2 = d2.contiguous()
        main_grad = getattr(table, "main_grad", None)
        if main_grad is not None:
            tgt, ret = main_grad, None
        else:
            tgt = torch.zeros(table.shape, dtype=torch.float32, device=table.device)
            ret = tgt
        rc = _lib.get_lib().mfb_embedding_bwd(flat.data_ptr(), d2.data_ptr(), tgt.data_ptr(), flat.numel(), H,
                                              int(ctx.vocab_start), table.shape[0], _lib.stream_ptr())
        _lib.check(rc, "mfb_embedding_bwd")
        _lib.count_launch()
        return None, (ret.to(table.dtype) if ret is not None else None), None


def embedding(ids: torch.Tensor, table: torch.Tensor, vocab_start: int = 0) -> torch.Tensor:
    """Row gather; ids outside ``[vocab_start, vocab_start + rows)`` give zero rows (vocab-parallel shard)."""
    if _on_gpu(table) and table.dtype == torch.bfloat16 and table.shape[1] % 8 == 0:
        return apply_fn(_EmbeddingFn, ids, table, vocab_start)
    local = ids - vocab_start
    ok = (local >= 0) & (local < table.shape[0])
    out = F.embedding(local.clamp(0, table.shape[0] - 1), table)
    return out * ok.unsqueeze(-1).to(out.dtype)


# =================================================================================================
# Cross-entropy (vocab-parallel aware)
# =================================================================================================
class _VocabParallelCERefFn(torch.autograd.Function):
    """Plain-PyTorch vocab-parallel cross-entropy with an explicit backward (softmax - onehot)."""

    @staticmethod
    def forward(ctx, logits, labels, vocab_start, group):
        lf = logits.float()
        m = lf.max(-1).values
        if group is not None:
            torch.distributed.all_reduce(m, op=torch.distributed.ReduceOp.MAX, group=group)
        e = (lf - m.unsqueeze(-1)).exp()
        s = e.sum(-1)
        local = labels - vocab_start
        ok = (local >= 0) & (local < lf.shape[-1])
        idx = local.clamp(0, lf.shape[-1] - 1)
        tgt = lf.gather(-1, idx.unsqueeze(-1)).squeeze(-1) * ok
        if group is not None:
            torch.distributed.all_reduce(s, group=group)
            torch.distributed.all_reduce(tgt, group=group)
        ctx.save_for_backward(e / s.unsqueeze(-1), idx, ok)
        ctx.in_dtype = logits.dtype
        return m + s.log() - tgt

    @staticmethod
    def backward(ctx, g):
        p, idx, ok = ctx.saved_tensors
        grad = p.clone()
        grad.scatter_add_(-1, idx.unsqueeze(-1), -ok.to(grad.dtype).unsqueeze(-1))
        return (grad * g.unsqueeze(-1)).to(ctx.in_dtype), None, None, None


def cross_entropy_reference(logits, labels, vocab_start=0, group=None):
    """Per-token NLL in fp32 from a (possibly vocab-sharded) logits tensor."""
    return _VocabParallelCERefFn.apply(logits, labels, vocab_start, group)


class _CrossEntropyFn(torch.autograd.Function):
    """Per-token loss; the backward pass overwrites the logits buffer with its gradient."""

    @staticmethod
    def forward(ctx, logits, labels, vocab_start, group):
        T, V = logits.shape
        lib = _lib.get_lib()
        dt = 0 if logits.dtype == torch.bfloat16 else 1
        stats = torch.empty((3, T), dtype=torch.float32, device=logits.device)
        labels = labels.to(torch.int64).contiguous()
        rc = lib.mfb_ce_stats(logits.data_ptr(), dt, labels.data_ptr(), stats[0].data_ptr(), stats[1].data_ptr(),
                              stats[2].data_ptr(), T, V, logits.stride(0), int(vocab_start), _lib.stream_ptr())
        _lib.check(rc, "mfb_ce_stats")
        _lib.count_launch()
        m, s, tgt = stats[0], stats[1], stats[2]
        if group is not None and torch.distributed.get_world_size(group) > 1:
            gm = m.clone()
            torch.distributed.all_reduce(gm, op=torch.distributed.ReduceOp.MAX, group=group)
            s = s * torch.exp(m - gm)
            st = torch.stack((s, tgt))
            torch.distributed.all_reduce(st, group=group)
            s, tgt, m = st[0], st[1], gm
        lse = m + torch.log(s)
        loss = lse - tgt
        ctx.save_for_backward(logits, labels, lse)
        ctx.vocab_start = vocab_start
        return loss

    @staticmethod
    def backward(ctx, dloss):
        logits, labels, lse = ctx.saved_tensors
        T, V = logits.shape
        dt = 0 if logits.dtype == torch.bfloat16 else 1
        g = dloss.float().contiguous()
        # the logits are dead after this point: reuse their storage for the gradient
        rc = _lib.get_lib().mfb_ce_bwd(logits.data_ptr(), logits.data_ptr(), dt, labels.data_ptr(),
                                       lse.data_ptr(), g.data_ptr(), T, V, logits.stride(0),
                                       int(ctx.vocab_start), _lib.stream_ptr())
        _lib.check(rc, "mfb_ce_bwd")
        _lib.count_launch()
        return logits, None, None, None


def cross_entropy(logits: torch.Tensor, labels: torch.Tensor, vocab_start: int = 0, group=None) -> torch.Tensor:
    """Per-token negative log-likelihood ``[T]`` (fp32). ``logits``: ``[T, V_local]``.

    On CUDA the backward pass writes the gradient into the storage of ``logits``; callers must not
    reuse the logits after calling ``backward``.
    """
    if _on_gpu(logits) and logits.dtype in (torch.bfloat16, torch.float32) and logits.stride(-1) == 1:
        return _CrossEntropyFn.apply(logits, labels, vocab_start, group)
    return cross_entropy_reference(logits, labels, vocab_start, group)


# =================================================================================================
# Attention
# =================================================================================================
def attention_reference(q, k, v, causal=True, scale=None, q_offset=0):
    """q: [B, Sq, Hq, D], k/v: [B, Sk, Hkv, D(v)] -> [B, Sq, Hq, Dv]; fp32 math; GQA by head repeat."""
    B, Sq, Hq, D = q.shape
    Hkv = k.shape[2]
    rep = Hq // Hkv
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if causal:
        Sk = k.shape[1]
        qi = torch.arange(Sq, device=q.device).unsqueeze(-1) + q_offset
        ki = torch.arange(Sk, device=q.device).unsqueeze(0)
        s = s.masked_fill(ki > qi, float("-inf"))
    p = torch.softmax(s, dim=-1)
    o = torch.matmul(p, vf)
    return o.permute(0, 2, 1, 3).to(q.dtype)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = True,
              scale: Optional[float] = None) -> torch.Tensor:
    """Dense (batched, equal-length) attention. q: ``[B,S,Hq,D]``, k/v: ``[B,S,Hkv,D]`` -> ``[B,S,Hq,Dv]``."""
    if _on_gpu(q):
        if _ATTN_BACKEND in ("auto", "native"):
            from . import attention as _attn
            if _attn.supported(q, k, v, causal):
                return _attn.flash_attention(q, k, v, causal, scale)
            if _ATTN_BACKEND == "native":
                raise _lib.KernelLibraryError("native attention kernel does not support this problem")
        Hq, Hkv = q.shape[2], k.shape[2]
        o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                           is_causal=causal, scale=scale, enable_gqa=(Hq != Hkv))
        return o.transpose(1, 2)
    return attention_reference(q, k, v, causal, scale)


# =================================================================================================
# Block-scaled fp8 (e4m3) GEMM: 1 x 128 activation scales, 128 x 128 weight scales (DeepSeek-V3 checkpoints)
# =================================================================================================
FP8_MAX = 448.0


def quantize_weight_128x128(w: torch.Tensor):
    """``w [N, K]`` (or ``[G, N, K]``) → ``(wq e4m3, scale_inv fp32 [.., N/128, K/128])`` with ``w ≈ wq * scale_inv`` per block
    (the layout of DeepSeek-V3 checkpoints: ``weight`` + ``weight_scale_inv``)."""
    lead = w.shape[:-2]
    N, K = w.shape[-2:]
    if N % 128 or K % 128:
        raise ValueError(f"weight [{N}, {K}] must be a multiple of 128 in both dimensions")
    blocks = w.float().reshape(*lead, N // 128, 128, K // 128, 128)
    amax = blocks.abs().amax(dim=(-3, -1), keepdim=True).clamp_min(1e-12)
    scale = amax / FP8_MAX
    q = (blocks / scale).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn).reshape(w.shape)
    return q, scale.reshape(*lead, N // 128, K // 128).contiguous()


def quantize_act_1x128(x: torch.Tensor):
    """``x [T, K]`` bf16 → ``(xq e4m3 [T, K], sa fp32 [K/128, T_pad])`` with one scale per row and block of 128
    (``T_pad`` = T rounded up to 128: the GEMM reads scales of whole row blocks)."""
    T, K = x.shape
    if K % 128:
        raise ValueError(f"K={K} must be a multiple of 128")
    Tp = (T + 127) // 128 * 128
    if _on_gpu(x) and x.dtype == torch.bfloat16:
        x = x.contiguous()
        q = torch.empty(T, K, dtype=torch.float8_e4m3fn, device=x.device)
        # scales of the rows between T and T_pad stay unwritten: they only meet the zero-filled operand rows of the
        # last row block, whose results are never stored
        sa = torch.empty(K // 128, Tp, dtype=torch.float32, device=x.device)
        rc = _lib.get_lib().mfb_quant_act_1x128(x.data_ptr(), x.stride(0), q.data_ptr(), K, sa.data_ptr(), Tp, T, K,
                                                _lib.stream_ptr())
        _lib.check(rc, "mfb_quant_act_1x128")
        _lib.count_launch()
        return q, sa
    b = x.float().reshape(T, K // 128, 128)
    amax = b.abs().amax(-1, keepdim=True)
    scale = torch.where(amax > 0, amax / FP8_MAX, torch.ones_like(amax))
    q = (b / scale).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn).reshape(T, K)
    sa = torch.ones(K // 128, Tp, dtype=torch.float32, device=x.device)
    sa[:, :T] = scale.squeeze(-1).t()
    return q, sa


def fp8_gemm_reference(xq, sa, wq, sb):
    """fp32 oracle: de-quantise both operands block by block and multiply. ``wq [N, K]``, ``sb [N/128, K/128]``."""
    T, K = xq.shape
    x = xq.float().reshape(T, K // 128, 128) * sa[:, :T].t().unsqueeze(-1)
    N = wq.shape[0]
    w = wq.float().reshape(N // 128, 128, K // 128, 128) * sb.reshape(N // 128, 1, K // 128, 1)
    return x.reshape(T, K) @ w.reshape(N, K).t()


FP8_DECODE_MAX_ROWS_PER_GROUP = 160     # grouped calls with at most this many (padded) rows per expert are "decode"
_FP8_DECODE_KERNEL = os.environ.get("MFB_FP8_DECODE_KERNEL", "1") != "0"


def fp8_gemm(xq: torch.Tensor, sa: torch.Tensor, wq: torch.Tensor, sb: torch.Tensor, *, block_group=None, num_blocks=None,
             group_offsets=None, seg_fill=None):
    """``y [T, N] (bf16) = dequant(xq, sa) @ dequant(wq, sb)^T``. Grouped form: ``wq [G, N, K]``, ``sb [G, N/128, K/128]``,
    rows of ``xq`` sorted by expert in 128-row blocks (``block_group`` / ``num_blocks`` as for ``grouped_gemm``).

    Two kernels: ``gemm_fp8.cu`` (128 token rows per tile) and, for at most 64 tokens or for grouped calls with a
    few rows per expert whose segment fill is known (``group_offsets`` / ``seg_fill`` of the expert plan),
    ``gemm_fp8_decode.cu`` (the weight on the MMA rows, 32 or 64 tokens per tile)."""
    T, K = xq.shape
    grouped = wq.dim() == 3
    G = wq.shape[0] if grouped else 1
    N = wq.shape[-2]
    if not _on_gpu(xq):
        if not grouped:
            return fp8_gemm_reference(xq, sa, wq, sb).to(torch.bfloat16)
        out = torch.zeros(T, N, dtype=torch.bfloat16, device=xq.device)
        nb = int(num_blocks.item())
        for i, g in enumerate(block_group[:nb].tolist()):
            rows = slice(i * 128, (i + 1) * 128)
            out[rows] = fp8_gemm_reference(xq[rows], sa[:, rows], wq[g], sb[g]).to(torch.bfloat16)
        return out
    out = torch.empty(T, N, dtype=torch.bfloat16, device=xq.device)
    st = _lib.status_word(xq.device)
    w2 = wq.reshape(G * N, K)
    lib = _lib.get_lib()
    decode = _FP8_DECODE_KERNEL and sa.stride(0) % 4 == 0 and (
        (not grouped and T <= 64) or
        (grouped and group_offsets is not None and seg_fill is not None and T % 128 == 0
         and T <= FP8_DECODE_MAX_ROWS_PER_GROUP * G))
    if decode:
        rc = lib.mfb_gemm_fp8_decode(
            xq.data_ptr(), w2.data_ptr(), out.data_ptr(), sa.data_ptr(), sa.stride(0), sb.contiguous().data_ptr(), T, N, K,
            xq.stride(0), w2.stride(0), out.stride(0), 1 if grouped else 0, G, _lib.ptr(block_group), _lib.ptr(num_blocks),
            _lib.ptr(group_offsets), _lib.ptr(seg_fill), st.data_ptr(), _lib.stream_ptr())
        _lib.check(rc, "mfb_gemm_fp8_decode")
        _lib.count_launch()
        return out
    rc = lib.mfb_gemm_fp8_blockscaled(
        xq.data_ptr(), w2.data_ptr(), out.data_ptr(), sa.data_ptr(), sa.stride(0), sb.contiguous().data_ptr(), T, N, K,
        xq.stride(0), w2.stride(0), out.stride(0), 1 if grouped else 0, G, _lib.ptr(block_group), _lib.ptr(num_blocks),
        st.data_ptr(), _lib.stream_ptr())
    _lib.check(rc, "mfb_gemm_fp8_blockscaled")
    _lib.count_launch()
    return out


def fp8_linear(x: torch.Tensor, wq: torch.Tensor, sb: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Inference linear layer on block-scaled fp8 weights: activations are quantised on the fly (1 x 128 blocks)."""
    shape = x.shape
    x2 = x.reshape(-1, shape[-1])
    xq, sa = quantize_act_1x128(x2.to(torch.bfloat16))
    y = fp8_gemm(xq, sa, wq, sb)
    if bias is not None:
        y = y + bias
    return y.reshape(*shape[:-1], wq.shape[-2]).to(x.dtype)


# =================================================================================================
# W8A8: int8 activations x int8 weights on the integer tensor-core path
# =================================================================================================
def quantize_act_int8(x: torch.Tensor, smooth: Optional[torch.Tensor] = None):
    """``x [T, K]`` → ``(int8 [T, K], scale fp32 [T])``: one scale per token, ``absmax / 127``; ``smooth [K]`` divides
    the activations first (SmoothQuant)."""
    T, K = x.shape
    if _on_gpu(x) and x.dtype == torch.bfloat16:
        x = x.contiguous()
        q = torch.empty(T, K, dtype=torch.int8, device=x.device)
        scale = torch.empty(T, dtype=torch.float32, device=x.device)
        sm = smooth.float().contiguous() if smooth is not None else None
        rc = _lib.get_lib().mfb_quant_act_int8(x.data_ptr(), x.stride(0), q.data_ptr(), K, scale.data_ptr(), _lib.ptr(sm),
                                               T, K, _lib.stream_ptr())
        _lib.check(rc, "mfb_quant_act_int8")
        _lib.count_launch()
        return q, scale
    xf = x.float() / smooth.float() if smooth is not None else x.float()
    amax = xf.abs().amax(-1)
    scale = torch.where(amax > 0, amax / 127.0, torch.ones_like(amax))
    q = torch.round(xf / scale.unsqueeze(-1)).clamp(-127, 127).to(torch.int8)
    return q, scale


def w8a8_gemm(xq: torch.Tensor, sa: torch.Tensor, wq: torch.Tensor, sb: torch.Tensor,
              bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``bf16(sa[m] * sb[n] * (xq @ wq^T)[m, n] + bias[n])`` with ``xq [M, K]``, ``wq [N, K]`` int8, int32 accumulation."""
    M, K = xq.shape
    N = wq.shape[0]
    if _on_gpu(xq) and K % 16 == 0 and N % 8 == 0:
        xq, wq = xq.contiguous(), wq.contiguous()
        out = torch.empty(M, N, dtype=torch.bfloat16, device=xq.device)
        b = bias.to(torch.bfloat16).contiguous() if bias is not None else None
        st = _lib.status_word(xq.device)
        rc = _lib.get_lib().mfb_gemm_w8a8(xq.data_ptr(), wq.data_ptr(), out.data_ptr(), sa.float().contiguous().data_ptr(),
                                          sb.float().contiguous().data_ptr(), _lib.ptr(b), M, N, K, K, K, N,
                                          st.data_ptr(), _lib.stream_ptr())
        _lib.check(rc, "mfb_gemm_w8a8")
        _lib.count_launch()
        return out
    # integer matmul on the CPU, double on a GPU whose shape the kernel does not take: both exact
    acc = (xq.double() @ wq.double().t()) if xq.is_cuda else (xq.to(torch.int64) @ wq.to(torch.int64).t())
    y = acc.float() * sa.float().unsqueeze(-1) * sb.float().unsqueeze(0)
    if bias is not None:
        y = y + bias.float()
    return y.to(torch.bfloat16)


def w8a8_linear(x: torch.Tensor, wq: torch.Tensor, sb: torch.Tensor, smooth: Optional[torch.Tensor] = None,
                bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Linear layer on int8 weights with dynamically quantised int8 activations (per token)."""
    shape = x.shape
    x2 = x.reshape(-1, shape[-1])
    xq, sa = quantize_act_int8(x2.to(torch.bfloat16) if x2.is_cuda else x2, smooth)
    y = w8a8_gemm(xq, sa, wq, sb.reshape(-1), bias)
    return y.reshape(*shape[:-1], wq.shape[0]).to(x.dtype)


# =================================================================================================
# MoE router
# =================================================================================================
def router_topk_reference(logits, bias, k, sigmoid, norm, scale, groups=0, group_topk=0):
    """PyTorch oracle of the router kernel: returns ``(probs [T,k], ids [T,k], scores [T,E])``."""
    scores = torch.sigmoid(logits) if sigmoid else torch.softmax(logits, dim=-1)
    sel = scores if bias is None else scores + bias
    T, E = scores.shape
    if groups and groups > 1 and group_topk and group_topk < groups:
        grouped = sel.view(T, groups, E // groups)
        if bias is not None:
            gscore = grouped.topk(min(2, E // groups), dim=-1).values.sum(-1)
        else:
            gscore = grouped.max(-1).values
        keep = gscore.topk(group_topk, dim=-1).indices
        mask = torch.zeros(T, groups, dtype=torch.bool, device=scores.device).scatter_(1, keep, True)
        sel = sel.masked_fill(~mask.unsqueeze(-1).expand(T, groups, E // groups).reshape(T, E), float("-inf"))
    ids = sel.topk(k, dim=-1).indices
    probs = scores.gather(1, ids)
    if norm:
        probs = probs / (probs.sum(-1, keepdim=True) + 1e-20)
    return probs * scale, ids, scores


class _RouterFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, bias, k, sigmoid, norm, scale, groups, group_topk, need_scores, counts):
        T, E = logits.shape
        logits = logits.contiguous()
        probs = torch.empty(T, k, dtype=torch.float32, device=logits.device)
        ids = torch.empty(T, k, dtype=torch.int64, device=logits.device)
        scores = torch.empty(T, E, dtype=torch.float32, device=logits.device) if need_scores else None
        rc = _lib.get_lib().mfb_router_fwd(logits.data_ptr(), _lib.ptr(bias), probs.data_ptr(), ids.data_ptr(),
                                           _lib.ptr(scores), _lib.ptr(counts), T, E, k, int(sigmoid), int(norm),
                                           int(groups or 0), int(group_topk or 0), float(scale), _lib.stream_ptr())
        _lib.check(rc, "mfb_router_fwd")
        _lib.count_launch()
        ctx.save_for_backward(logits, ids)
        ctx.cfg = (k, sigmoid, norm, scale)
        ctx.mark_non_differentiable(ids)
        if scores is None:
            scores = torch.empty(0, device=logits.device)
            ctx.no_scores = True
        else:
            ctx.no_scores = False
        return probs, ids, scores

    @staticmethod
    def backward(ctx, dprobs, _dids, dscores):
        logits, ids = ctx.saved_tensors
        k, sigmoid, norm, scale = ctx.cfg
        T, E = logits.shape
        dlogits = torch.empty_like(logits)
        ds = None if ctx.no_scores or dscores is None else dscores.contiguous().float()
        rc = _lib.get_lib().mfb_router_bwd(logits.data_ptr(), ids.data_ptr(), dprobs.contiguous().float().data_ptr(),
                                           _lib.ptr(ds), dlogits.data_ptr(), T, E, k, int(sigmoid), int(norm),
                                           float(scale), _lib.stream_ptr())
        _lib.check(rc, "mfb_router_bwd")
        _lib.count_launch()
        return (dlogits,) + (None,) * 9


def router_topk(logits: torch.Tensor, bias: Optional[torch.Tensor], k: int, *, sigmoid: bool = False, norm: bool = True,
                scale: float = 1.0, groups: int = 0, group_topk: int = 0, need_scores: bool = False,
                counts: Optional[torch.Tensor] = None):
    """Fused router: ``(probs [T,k] fp32, ids [T,k] int64, scores [T,E] | None)``; ``counts [E]`` (fp32) is
    incremented by the number of copies routed to each expert."""
    E = logits.shape[-1]
    if _on_gpu(logits) and logits.dtype == torch.float32 and E <= 512 and k <= 32 and (not groups or groups <= 32):
        probs, ids, scores = apply_fn(_RouterFn, logits, bias, k, sigmoid, norm, scale, groups, group_topk, need_scores, counts)
        return probs, ids, (scores if need_scores else None)
    probs, ids, scores = router_topk_reference(logits.float(), bias, k, sigmoid, norm, scale, groups, group_topk)
    if counts is not None:
        counts.scatter_add_(0, ids.reshape(-1), torch.ones(ids.numel(), dtype=counts.dtype, device=counts.device))
    return probs, ids, (scores if need_scores else None)


# =================================================================================================
# Optimizer helpers
# =================================================================================================
def grad_sumsq(g: torch.Tensor, out: torch.Tensor, accumulate: bool = False):
    """``out (+)= sum(g^2)`` for a flat bf16/fp32 buffer; ``out`` is a 1-element fp32 tensor."""
    if not _on_gpu(g):
        val = g.float().pow(2).sum()
        if accumulate:
            out.add_(val)
        else:
            out.copy_(val.reshape(out.shape))
        return out
    lib = _lib.get_lib()
    scratch = _scratch(g.device, lib.mfb_grad_sumsq_scratch())
    dt = 0 if g.dtype == torch.bfloat16 else 1
    rc = lib.mfb_grad_sumsq(g.data_ptr(), dt, g.numel(), scratch.data_ptr(), out.data_ptr(), int(accumulate),
                            _lib.stream_ptr())
    _lib.check(rc, "mfb_grad_sumsq")
    _lib.count_launch(2)
    return out


def split_master(master: torch.Tensor, p: torch.Tensor, lo: torch.Tensor):
    """``(p, lo) <- master`` so that ``join_master`` gives the fp32 value back exactly.

    ``p`` is bf16 (the master rounded to nearest, ties up in magnitude), ``lo`` is int16 with
    ``master_bits = (p_bits << 16) + lo``.
    """
    if not _on_gpu(master):
        bits = master.contiguous().view(torch.int32)
        hi = (bits + 0x8000) >> 16          # round half up on the magnitude bits
        p.copy_(hi.to(torch.int16).view(torch.bfloat16))
        lo.copy_((bits - (hi << 16)).to(torch.int16))
        return
    rc = _lib.get_lib().mfb_split_master(master.data_ptr(), p.data_ptr(), lo.data_ptr(), master.numel(),
                                         _lib.stream_ptr())
    _lib.check(rc, "mfb_split_master")
    _lib.count_launch()


def join_master(p: torch.Tensor, lo: torch.Tensor) -> torch.Tensor:
    master = torch.empty(p.shape, dtype=torch.float32, device=p.device)
    if not _on_gpu(p):
        hi = p.view(torch.int16).to(torch.int32) << 16
        lov = lo.view(torch.int16).to(torch.int32)
        master.copy_((hi + lov).view(torch.float32))
        return master
    rc = _lib.get_lib().mfb_join_master(p.data_ptr(), lo.data_ptr(), master.data_ptr(), p.numel(),
                                        _lib.stream_ptr())
    _lib.check(rc, "mfb_join_master")
    _lib.count_launch()
    return master


def adamw_step(p, lo, m, v, g, *, lr, beta1, beta2, eps, weight_decay, step, decay_end=None,
               sumsq=None, skipped=None, max_norm=0.0, skip_threshold=0.0, grad_scale=1.0):
    """One fused AdamW update of a flat shard (see ``loss_optim.cu``). CPU body mirrors the kernel."""
    n = p.numel()
    decay_end = n if decay_end is None else decay_end
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    if _on_gpu(p):
        gd = 0 if g.dtype == torch.bfloat16 else 1
        rc = _lib.get_lib().mfb_adamw(p.data_ptr(), lo.data_ptr(), m.data_ptr(), v.data_ptr(), g.data_ptr(), gd,
                                      _lib.ptr(sumsq), _lib.ptr(skipped), n, decay_end, lr, beta1, beta2, eps,
                                      weight_decay, bc1, bc2, max_norm, skip_threshold, grad_scale,
                                      _lib.stream_ptr())
        _lib.check(rc, "mfb_adamw")
        _lib.count_launch()
        return
    clip = grad_scale
    if sumsq is not None:
        ss = float(sumsq)
        nrm = math.sqrt(ss) * abs(grad_scale) if math.isfinite(ss) and ss >= 0 else float("inf")
        if not math.isfinite(ss) or (skip_threshold > 0 and nrm >= skip_threshold):
            if skipped is not None:
                skipped.fill_(1)
            return
        if max_norm > 0 and nrm >= max_norm:
            clip *= max_norm / (nrm + 1e-6)
    w = join_master(p, lo)
    gr = g.float() * clip
    m.mul_(beta1).add_(gr, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(gr, gr, value=1 - beta2)
    w[:decay_end] *= (1 - lr * weight_decay)
    w -= (lr / bc1) * m / ((v / bc2).sqrt() + eps)
    split_master(w, p, lo)
