"""The allocation-free RMSNorm backward must agree with the regular entry point.

Some users of the kernel library cannot allocate device memory at the point where they need this
kernel (a host application that owns all GPU memory, a serving loop that has frozen its allocator, a
stream under capture). For them the library exports ``mfb_rmsnorm_bwd_noalloc``, which keeps its partial
sums in an array compiled into the library. This test calls that symbol directly through ctypes, twice in
a row with different data (the array is shared between calls and keeps old contents, so the second call
shows that stale partial sums do not leak into the result), and compares with ``mfb_rmsnorm_bwd``.
The file name sorts last on purpose: a failure here cannot hide the result of any other test.
"""
import ctypes

import pytest
import torch

from mindformers_b200.ops import _lib

pytestmark = pytest.mark.gpu


def _bind(lib):
    fn = lib.mfb_rmsnorm_bwd_noalloc
    P, I = ctypes.c_void_p, ctypes.c_int
    fn.argtypes = [P, P, P, P, P, P, P, P, I, I, I, P]
    fn.restype = I
    return fn


def _case(T, H, seed, with_res):
    g = torch.Generator(device="cuda").manual_seed(seed)
    dy = torch.randn(T, H, device="cuda", generator=g).to(torch.bfloat16)
    h = torch.randn(T, H, device="cuda", generator=g).to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(H, device="cuda", generator=g)).to(torch.bfloat16)
    rstd = torch.rsqrt(h.float().pow(2).mean(-1) + 1e-5).contiguous()
    dres = torch.randn(T, H, device="cuda", generator=g).to(torch.bfloat16) if with_res else None
    return dy, h, w, rstd, dres


def test_noalloc_entry_matches_regular_entry_twice_in_a_row():
    lib = _lib.get_lib()
    noalloc = _bind(lib)
    stream = _lib.stream_ptr()
    # second case is smaller in both dimensions: rows and columns written by the first call stay in the array
    for T, H, seed, with_res in [(700, 4096, 1, True), (37, 2048, 2, False)]:
        dy, h, w, rstd, dres = _case(T, H, seed, with_res)
        dx_a, dx_b = torch.empty_like(h), torch.empty_like(h)
        dw_a = torch.empty(H, device="cuda", dtype=torch.float32)
        dw_b = torch.empty(H, device="cuda", dtype=torch.float32)
        parts = lib.mfb_rmsnorm_bwd_parts(T)
        scratch = torch.empty(parts * H, device="cuda", dtype=torch.float32)
        rc = lib.mfb_rmsnorm_bwd(dy.data_ptr(), h.data_ptr(), w.data_ptr(), rstd.data_ptr(), _lib.ptr(dres),
                                 dx_a.data_ptr(), dw_a.data_ptr(), 0, 0, scratch.data_ptr(), T, H, stream)
        assert rc == 0, lib.mfb_last_error()
        rc = noalloc(dy.data_ptr(), h.data_ptr(), w.data_ptr(), rstd.data_ptr(), _lib.ptr(dres), dx_b.data_ptr(),
                     dw_b.data_ptr(), 0, 0, T, H, stream)
        assert rc == 0, lib.mfb_last_error()
        torch.cuda.synchronize()
        assert torch.equal(dx_a, dx_b)
        err = ((dw_a - dw_b).norm() / (dw_a.norm() + 1e-12)).item()
        assert err < 1e-2, err


def _fp32_reference(dy, h, w, rstd, dres):
    """dx and dw of RMSNorm in fp32 from the same saved statistics."""
    dyf, hf, wf = dy.float(), h.float(), w.float()
    xhat = hf * rstd[:, None]
    dw = (dyf * xhat).sum(0)
    g = dyf * wf
    dx = rstd[:, None] * (g - xhat * (g * xhat).mean(-1, keepdim=True))
    if dres is not None:
        dx = dx + dres.float()
    return dx, dw


@pytest.mark.parametrize("T,H,with_res", [(300, 8192, True), (5000, 8192, False), (149, 1024, True)])
def test_noalloc_entry_at_its_widest_row_and_accumulating_against_fp32(T, H, with_res):
    """H = 8192 is the documented maximum; T > 148 makes every thread block walk several rows; ``accumulate = 1`` adds
    onto a weight gradient that is already there. Checked against an fp32 evaluation, twice in a row."""
    lib = _lib.get_lib()
    noalloc = _bind(lib)
    stream = _lib.stream_ptr()
    for seed in (11, 12):
        dy, h, w, rstd, dres = _case(T, H, seed, with_res)
        dx = torch.empty_like(h)
        base = torch.randn(H, device="cuda", dtype=torch.float32)
        dw = base.clone()
        rc = noalloc(dy.data_ptr(), h.data_ptr(), w.data_ptr(), rstd.data_ptr(), _lib.ptr(dres), dx.data_ptr(),
                     dw.data_ptr(), 0, 1, T, H, stream)
        assert rc == 0, lib.mfb_last_error()
        torch.cuda.synchronize()
        dx_ref, dw_ref = _fp32_reference(dy, h, w, rstd, dres)
        assert ((dx.float() - dx_ref).norm() / dx_ref.norm()).item() < 5e-3          # bf16 rounding of dx
        assert (((dw - base) - dw_ref).norm() / dw_ref.norm()).item() < 1e-4         # fp32 sums in another order


def test_noalloc_entry_rejects_rows_wider_than_its_scratch():
    lib = _lib.get_lib()
    noalloc = _bind(lib)
    t = torch.zeros(8, device="cuda")
    rc = noalloc(t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), 0, t.data_ptr(), t.data_ptr(), 0, 0, 1,
                 16384, _lib.stream_ptr())
    assert rc == 1
    assert b"at most 8192" in lib.mfb_last_error()
