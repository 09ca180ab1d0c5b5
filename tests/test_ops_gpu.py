"""Numerics of the sm_100a kernels against plain PyTorch fp32 references of the same op."""
import math

import pytest
import torch

from mindformers_b200.ops import _lib
from mindformers_b200.ops import functional as Fn

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rel_err(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


def _status_ok():
    assert _lib.read_status() == 0, "a bounded device wait ran out"


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (4096, 6144, 4096), (300, 384, 200),
                                   (64, 128, 128), (1000, 3072, 1024), (128, 128, 64)])
def test_gemm_tn(M, N, K):
    torch.manual_seed(0)
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(N, K, device=DEV, dtype=torch.bfloat16)
    d = Fn.gemm(a, b)
    ref = a.float() @ b.float().t()
    torch.cuda.synchronize()
    _status_ok()
    assert _rel_err(d, ref) < 5e-3


@pytest.mark.parametrize("M,N,K", [(256, 512, 256), (4096, 4096, 6144), (384, 256, 192)])
def test_gemm_b_mn_major(M, N, K):
    torch.manual_seed(1)
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(K, N, device=DEV, dtype=torch.bfloat16)
    d = Fn.gemm(a, b, b_mn=True)
    ref = a.float() @ b.float()
    torch.cuda.synchronize()
    _status_ok()
    assert _rel_err(d, ref) < 5e-3


@pytest.mark.parametrize("M,N,K", [(256, 512, 256), (6144, 4096, 4096), (384, 256, 320)])
def test_gemm_both_mn_major(M, N, K):
    torch.manual_seed(2)
    a = torch.randn(K, M, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(K, N, device=DEV, dtype=torch.bfloat16)
    d = Fn.gemm(a, b, a_mn=True, b_mn=True, out_dtype=torch.float32)
    ref = a.float().t() @ b.float()
    torch.cuda.synchronize()
    _status_ok()
    assert _rel_err(d, ref) < 5e-3
    # accumulate twice into an fp32 buffer through the TMA reduce-add epilogue
    acc = torch.zeros(M, N, device=DEV, dtype=torch.float32)
    Fn.gemm(a, b, a_mn=True, b_mn=True, out=acc, accumulate=True)
    Fn.gemm(a, b, a_mn=True, b_mn=True, out=acc, accumulate=True)
    torch.cuda.synchronize()
    assert _rel_err(acc, 2 * ref) < 5e-3


@pytest.mark.parametrize("M,N,K,sm_limit", [(4096, 4096, 1024, 0), (1280, 256, 2048, 8), (1304, 520, 2056, 8),
                                            (768, 768, 512, 4)])
@pytest.mark.parametrize("layout", ["tn", "nn", "tt_f32"])
def test_gemm_pair_tail_split_matches_unsplit(M, N, K, sm_limit, layout):
    """CTA-pair GEMM: the K split of the tail wave (partials through the workspace) against fp32 matmul and
    against the same kernel without the split; run twice so that the second call meets re-armed flags."""
    torch.manual_seed(7)
    a_mn, b_mn = layout == "tt_f32", layout != "tn"
    a = torch.randn((K, M) if a_mn else (M, K), device=DEV, dtype=torch.bfloat16)
    b = torch.randn((K, N) if b_mn else (N, K), device=DEV, dtype=torch.bfloat16)
    ref = (a.float().t() if a_mn else a.float()) @ (b.float() if b_mn else b.float().t())
    odt = torch.float32 if layout == "tt_f32" else torch.bfloat16
    try:
        Fn.set_pair_gemm(True, 1)
        plain = Fn.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out_dtype=odt, sm_limit=sm_limit)
        Fn.set_pair_gemm(True, 4)
        for _ in range(2):
            split = Fn.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out_dtype=odt, sm_limit=sm_limit)
            torch.cuda.synchronize()
            _status_ok()
            assert _rel_err(split, ref) < 5e-3
            assert _rel_err(split, plain) < 2e-3
        assert _rel_err(plain, ref) < 5e-3
    finally:
        Fn.set_pair_gemm(True, 4)


def test_gemm_pair_matches_single_cta_kernel():
    torch.manual_seed(8)
    a = torch.randn(1024, 1536, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(2048, 1536, device=DEV, dtype=torch.bfloat16)
    try:
        Fn.set_pair_gemm(False)
        single = Fn.gemm(a, b)
        Fn.set_pair_gemm(True, 1)
        pair = Fn.gemm(a, b)
    finally:
        Fn.set_pair_gemm(True, 4)
    torch.cuda.synchronize()
    _status_ok()
    assert torch.equal(single, pair), "same K order per output element: the two tilings must agree bitwise"


def test_linear_autograd_matches_torch():
    torch.manual_seed(3)
    x = torch.randn(512, 1024, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    w = torch.randn(768, 1024, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    y = Fn.linear(x, w)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    wr = w.detach().float().requires_grad_()
    yr = xr @ wr.t()
    yr.backward(g.float())
    assert _rel_err(y, yr) < 5e-3
    assert _rel_err(x.grad, xr.grad) < 5e-3
    assert _rel_err(w.grad, wr.grad) < 5e-3


def test_grouped_gemm_and_wgrad():
    torch.manual_seed(4)
    G, K, N = 4, 256, 384
    counts = [128, 0, 384, 256]
    offs = [0]
    for c in counts:
        offs.append(offs[-1] + c)
    R = offs[-1] + 256  # spare rows beyond the used blocks
    a = torch.randn(R, K, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(G, N, K, device=DEV, dtype=torch.bfloat16)
    bg = []
    for g, c in enumerate(counts):
        bg += [g] * (c // 128)
    nb = len(bg)
    block_group = torch.tensor(bg + [0] * (R // 128 - nb), device=DEV, dtype=torch.int32)
    num_blocks = torch.tensor([nb], device=DEV, dtype=torch.int32)
    out = Fn.grouped_gemm(a, b, block_group, num_blocks)
    torch.cuda.synchronize()
    _status_ok()
    for g in range(G):
        rows = slice(offs[g], offs[g + 1])
        if counts[g]:
            assert _rel_err(out[rows], a[rows].float() @ b[g].float().t()) < 5e-3
    # dgrad: dy [R,N] x W[g] [N,K] -> [R,K]
    dy = torch.randn(R, N, device=DEV, dtype=torch.bfloat16)
    dx = Fn.grouped_gemm(dy, b, block_group, num_blocks, b_mn=True)
    torch.cuda.synchronize()
    _status_ok()
    for g in range(G):
        rows = slice(offs[g], offs[g + 1])
        if counts[g]:
            assert _rel_err(dx[rows], dy[rows].float() @ b[g].float()) < 5e-3
    # wgrad per expert (expert 1 is empty and must come out as zeros)
    go = torch.tensor(offs, device=DEV, dtype=torch.int32)
    dw = torch.full((G, N, K), 7.0, device=DEV, dtype=torch.float32)
    Fn.grouped_wgrad(dy, a, go, G, dw)
    torch.cuda.synchronize()
    _status_ok()
    for g in range(G):
        rows = slice(offs[g], offs[g + 1])
        ref = dy[rows].float().t() @ a[rows].float()
        if counts[g]:
            assert _rel_err(dw[g], ref) < 5e-3
        else:
            assert dw[g].abs().max().item() == 0.0


@pytest.mark.parametrize("T,H", [(64, 4096), (33, 2048), (17, 7168), (5, 512)])
def test_rmsnorm_fwd_bwd(T, H):
    torch.manual_seed(5)
    x = torch.randn(T, H, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    r = torch.randn(T, H, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    w = (1 + 0.1 * torch.randn(H, device=DEV)).to(torch.bfloat16).requires_grad_()
    y, h = Fn.rmsnorm(x, w, 1e-5, residual=r)
    gy, gh = torch.randn_like(y), torch.randn_like(h)
    (y * gy).sum().backward(retain_graph=True)
    (h * gh).sum().backward()
    xr, rr, wr = (t.detach().float().requires_grad_() for t in (x, r, w))
    hr = (xr + rr).to(torch.bfloat16).float() + 0 * (xr + rr)  # value rounded like the kernel, grad identity
    hr = (xr + rr) + ((xr + rr).to(torch.bfloat16).float() - (xr + rr)).detach()
    yr = hr * torch.rsqrt(hr.pow(2).mean(-1, keepdim=True) + 1e-5) * wr
    ((yr * gy.float()).sum() + (hr * gh.float()).sum()).backward()
    assert _rel_err(y, yr) < 1e-2
    assert _rel_err(x.grad, xr.grad) < 1e-2
    assert _rel_err(r.grad, rr.grad) < 1e-2
    assert _rel_err(w.grad, wr.grad) < 1e-2


def test_swiglu_fwd_bwd():
    torch.manual_seed(6)
    x = torch.randn(257, 2 * 1536, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    y = Fn.swiglu(x)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    a, b = xr.chunk(2, -1)
    yr = torch.nn.functional.silu(a) * b
    yr.backward(g.float())
    assert _rel_err(y, yr) < 1e-2
    assert _rel_err(x.grad, xr.grad) < 1e-2


@pytest.mark.parametrize("interleaved", [False, True])
def test_rope(interleaved):
    torch.manual_seed(7)
    T, nq, nkv, hd = 96, 8, 2, 128
    heads = nq + 2 * nkv
    x0 = torch.randn(T, heads, hd, device=DEV, dtype=torch.bfloat16)
    inv = 1.0 / (10000 ** (torch.arange(0, hd, 2, device=DEV).float() / hd))
    ang = torch.arange(128, device=DEV).float()[:, None] * inv[None]
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    pos = torch.randint(0, 128, (T,), device=DEV)
    x = x0.clone().requires_grad_()
    y = Fn.rope(x * 1.0, cos, sin, pos, nq + nkv, hd, interleaved)
    ref = Fn.rope_reference(x0, cos, sin, pos, nq + nkv, hd, interleaved)
    assert _rel_err(y, ref) < 1e-2
    g = torch.randn_like(y)
    y.backward(g)
    x2 = x0.clone().float().requires_grad_()
    Fn.rope_reference(x2, cos, sin, pos, nq + nkv, hd, interleaved).backward(g.float())
    assert _rel_err(x.grad, x2.grad) < 1e-2


@pytest.mark.parametrize("V", [1024, 128256, 50001])
def test_cross_entropy(V):
    torch.manual_seed(8)
    T = 64
    logits = (torch.randn(T, V, device=DEV) * 2).to(torch.bfloat16)
    labels = torch.randint(0, V, (T,), device=DEV)
    lr = logits.detach().float().requires_grad_()
    ref = torch.nn.functional.cross_entropy(lr, labels, reduction="none")
    w = torch.rand(T, device=DEV)
    (ref * w).sum().backward()
    lg = logits.clone().requires_grad_()
    loss = Fn.cross_entropy(lg, labels)
    assert torch.allclose(loss, ref, atol=2e-3, rtol=2e-3)
    (loss * w).sum().backward()
    assert _rel_err(lg.grad, lr.grad) < 1e-2


def test_embedding():
    torch.manual_seed(9)
    V, H, T = 1000, 256, 333
    table = torch.randn(V, H, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    ids = torch.randint(0, V, (T,), device=DEV)
    out = Fn.embedding(ids, table)
    assert torch.equal(out, table[ids])
    g = torch.randn_like(out)
    out.backward(g)
    ref = torch.zeros(V, H, device=DEV)
    ref.index_add_(0, ids, g.float())
    assert _rel_err(table.grad, ref) < 1e-2


def test_adamw_matches_reference_and_master_is_exact():
    torch.manual_seed(10)
    n = 100003
    w = torch.randn(n, device=DEV) * 0.02
    p = torch.empty(n, device=DEV, dtype=torch.bfloat16)
    lo = torch.empty(n, device=DEV, dtype=torch.int16)
    Fn.split_master(w, p, lo)
    assert torch.equal(Fn.join_master(p, lo), w)
    m = torch.zeros(n, device=DEV)
    v = torch.zeros(n, device=DEV)
    wr, mr, vr = w.clone(), m.clone(), v.clone()
    sumsq = torch.zeros(1, device=DEV)
    for step in range(1, 4):
        g = torch.randn(n, device=DEV)
        Fn.grad_sumsq(g, sumsq)
        assert abs(sumsq.item() - g.pow(2).sum().item()) / g.pow(2).sum().item() < 1e-4
        Fn.adamw_step(p, lo, m, v, g, lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=step,
                      decay_end=n // 2, sumsq=sumsq, max_norm=1.0)
        nrm = g.norm()
        gc = g * min(1.0, 1.0 / (nrm.item() + 1e-6))
        mr = 0.9 * mr + 0.1 * gc
        vr = 0.95 * vr + 0.05 * gc * gc
        wr[: n // 2] *= 1 - 1e-3 * 0.1
        wr -= (1e-3 / (1 - 0.9 ** step)) * mr / ((vr / (1 - 0.95 ** step)).sqrt() + 1e-8)
    got = Fn.join_master(p, lo)
    assert torch.allclose(got, wr, atol=1e-6, rtol=1e-4)
    assert torch.allclose(p.float(), got, atol=0, rtol=2 ** -8)


@pytest.mark.parametrize("B,S,nq,nkv,causal", [(1, 128, 2, 1, True), (2, 512, 4, 2, True), (1, 1024, 8, 2, True),
                                               (1, 384, 2, 2, False), (1, 4096, 32, 8, True), (2, 2048, 16, 4, True),
                                               (1, 640, 4, 4, True)])
def test_flash_attention_fwd_bwd(B, S, nq, nkv, causal):
    from mindformers_b200.ops import attention as A
    torch.manual_seed(12)
    hd = 128
    packed = (torch.randn(B * S, nq + 2 * nkv, hd, device=DEV) * 0.5).to(torch.bfloat16).requires_grad_()
    out = A.flash_attention_packed(packed, B, S, nq, nkv, causal=causal)
    g = (torch.randn_like(out) * 0.1)
    out.backward(g)
    torch.cuda.synchronize()
    _status_ok()
    ref_in = packed.detach().float().requires_grad_()
    q = ref_in[:, :nq].reshape(B, S, nq, hd)
    k = ref_in[:, nq:nq + nkv].reshape(B, S, nkv, hd)
    v = ref_in[:, nq + nkv:].reshape(B, S, nkv, hd)
    ref = Fn.attention_reference(q, k, v, causal=causal).reshape(B * S, nq * hd)
    ref.backward(g.float())
    assert _rel_err(out, ref) < 1e-2
    gq, rq = packed.grad[:, :nq], ref_in.grad[:, :nq]
    gk, rk = packed.grad[:, nq:nq + nkv], ref_in.grad[:, nq:nq + nkv]
    gv, rv = packed.grad[:, nq + nkv:], ref_in.grad[:, nq + nkv:]
    assert _rel_err(gv, rv) < 2e-2
    assert _rel_err(gk, rk) < 2e-2
    assert _rel_err(gq, rq) < 2e-2


@pytest.mark.parametrize("B,S,nq,nkv,bounds", [
    (1, 1024, 4, 2, [0, 100, 130, 600, 1024]),          # documents that start and end inside tiles
    (2, 512, 4, 4, [0, 128, 256, 512]),                 # boundaries on tile edges
    (1, 640, 8, 2, [0, 640]),                           # one document: must equal the plain kernel
    (1, 2048, 8, 2, [0, 7, 8, 900, 1500, 1501, 2048]),  # very short documents next to long ones
])
def test_flash_attention_packed_sequences_match_per_document_attention(B, S, nq, nkv, bounds):
    """Packed rows (several documents per sequence, the layout of EOD-reset pre-training data): forward and backward of
    the kernels with document tables against fp32 attention evaluated separately on every document."""
    from mindformers_b200.ops import attention as A
    torch.manual_seed(len(bounds) + S)
    hd = 128
    packed = (torch.randn(B * S, nq + 2 * nkv, hd, device=DEV) * 0.5).to(torch.bfloat16).requires_grad_()
    cu = torch.tensor(bounds, device=DEV, dtype=torch.int32)
    asl = torch.full((B, 8), S, device=DEV, dtype=torch.int32)
    asl[:, :len(bounds) - 1] = cu[1:]
    doc_start, doc_end = A.document_tables(actual_seq_len=asl, B=B, S=S)
    out = A.flash_attention_packed(packed, B, S, nq, nkv, causal=True, doc_start=doc_start, doc_end=doc_end)
    g = (torch.randn_like(out) * 0.1)
    out.backward(g)
    torch.cuda.synchronize()
    _status_ok()
    ref_in = packed.detach().float().requires_grad_()
    r3 = ref_in.view(B, S, nq + 2 * nkv, hd)
    pieces = []
    for a, b in zip(bounds[:-1], bounds[1:]):
        if b > a:
            q, k, v = r3[:, a:b, :nq], r3[:, a:b, nq:nq + nkv], r3[:, a:b, nq + nkv:]
            pieces.append(Fn.attention_reference(q, k, v, causal=True))
    ref = torch.cat(pieces, dim=1).reshape(B * S, nq * hd)
    ref.backward(g.float())
    assert _rel_err(out, ref) < 1e-2
    for lo, hi in ((0, nq), (nq, nq + nkv), (nq + nkv, nq + 2 * nkv)):
        assert _rel_err(packed.grad[:, lo:hi], ref_in.grad[:, lo:hi]) < 2e-2
    if len(bounds) == 2:
        plain = A.flash_attention_packed(packed.detach(), B, S, nq, nkv, causal=True)
        assert torch.equal(plain, out.detach())


@pytest.mark.parametrize("split", [1, 2, 4])
@pytest.mark.parametrize("variant", [1, 2])
def test_flash_attention_backward_variants_and_group_split(variant, split):
    """Both backward kernels, and the pipelined one with a KV head's query-head group cut over 1 / 2 / 4 CTAs (fp32
    reduce-add of dK / dV), against fp32 attention."""
    from mindformers_b200.ops import attention as A
    if variant == 1 and split != 1:
        pytest.skip("the serial kernel has no group split")
    lib = _lib.get_lib()
    torch.manual_seed(40 + split)
    B, S, nq, nkv, hd = 2, 640, 8, 2, 128
    packed = (torch.randn(B * S, nq + 2 * nkv, hd, device=DEV) * 0.5).to(torch.bfloat16).requires_grad_()
    try:
        lib.mfb_flash_attn_set_bwd_variant(variant)
        lib.mfb_flash_attn_bwd2_set_split(split)
        out = A.flash_attention_packed(packed, B, S, nq, nkv, causal=True)
        g = (torch.randn_like(out) * 0.1)
        out.backward(g)
        torch.cuda.synchronize()
    finally:
        lib.mfb_flash_attn_set_bwd_variant(2)
        lib.mfb_flash_attn_bwd2_set_split(0)
    _status_ok()
    ref_in = packed.detach().float().requires_grad_()
    q = ref_in[:, :nq].reshape(B, S, nq, hd)
    k = ref_in[:, nq:nq + nkv].reshape(B, S, nkv, hd)
    v = ref_in[:, nq + nkv:].reshape(B, S, nkv, hd)
    ref = Fn.attention_reference(q, k, v, causal=True).reshape(B * S, nq * hd)
    ref.backward(g.float())
    assert _rel_err(out, ref) < 1e-2
    for lo, hi in ((0, nq), (nq, nq + nkv), (nq + nkv, nq + 2 * nkv)):
        assert _rel_err(packed.grad[:, lo:hi], ref_in.grad[:, lo:hi]) < 2e-2


@pytest.mark.parametrize("E,k,sig,groups,gk,bias", [(128, 8, False, 0, 0, False), (256, 8, True, 8, 4, True),
                                                    (64, 6, True, 0, 0, False), (160, 4, False, 4, 2, False)])
def test_router_topk_fwd_bwd(E, k, sig, groups, gk, bias):
    torch.manual_seed(E + k)
    T = 777
    logits = torch.randn(T, E, device="cuda") * 2.0
    b = (torch.randn(E, device="cuda") * 0.1) if bias else None
    la, lb = logits.clone().requires_grad_(), logits.clone().requires_grad_()
    counts = torch.zeros(E, device="cuda")
    p, ids, sc = Fn.router_topk(la, b, k, sigmoid=sig, norm=True, scale=2.5, groups=groups, group_topk=gk,
                               need_scores=True, counts=counts)
    pr, idr, scr = Fn.router_topk_reference(lb, b, k, sig, True, 2.5, groups, gk)
    assert torch.equal(ids.sort(-1).values, idr.sort(-1).values)
    assert torch.allclose(p.sort(-1).values, pr.sort(-1).values, rtol=1e-4, atol=1e-6)
    assert torch.allclose(sc, scr, rtol=1e-4, atol=1e-7)
    want = torch.zeros(E, device="cuda").scatter_add_(0, idr.reshape(-1), torch.ones(T * k, device="cuda"))
    assert torch.equal(counts, want)
    w = torch.randn(T, k, device="cuda")
    ws = torch.randn(T, E, device="cuda") * 0.1
    # same weights on matching experts: order the reference's columns like the kernel's
    order = torch.argsort(idr, -1).gather(1, torch.argsort(torch.argsort(ids, -1), -1))
    ((p * w).sum() + (sc * ws).sum()).backward()
    ((pr.gather(1, order) * w).sum() + (scr * ws).sum()).backward()
    assert torch.allclose(la.grad, lb.grad, rtol=2e-3, atol=2e-6)


def test_moe_exchange_kernels_match_torch_permute_single_rank():
    """ep = 1: rank/plan/scatter/gather kernels against the index-based PyTorch permutation, forward and backward."""
    from mindformers_b200.parallel import fused_comm
    from mindformers_b200.parallel.layers.moe import MoELayer
    from mindformers_b200.parallel.transformer_config import TransformerConfig
    torch.manual_seed(3)
    cfg = TransformerConfig(num_layers=1, hidden_size=256, num_attention_heads=4, ffn_hidden_size=512, num_moe_experts=8,
                            moe_router_topk=2, moe_ffn_hidden_size=128, params_dtype=torch.bfloat16, compute_dtype=torch.bfloat16,
                            moe_aux_loss_coeff=1e-2)
    cfg.device = "cuda"
    layer = MoELayer(cfg).train()
    x = (torch.randn(300, 256, device="cuda") * 0.5).to(torch.bfloat16)
    outs = []
    for fused in (True, False):
        cfg.fused_moe_comm = fused
        xi = x.clone().requires_grad_()
        for p in layer.parameters():
            p.grad = None
        y, aux = layer(xi)
        (y.float().pow(2).mean() + aux).backward()
        outs.append((y.detach().float(), xi.grad.float(), layer.router.weight.grad.float().clone(),
                     layer.experts.weight1.grad.float().clone()))
    for a, b in zip(*outs):
        assert torch.allclose(a, b, rtol=3e-2, atol=3e-3), (a - b).abs().max()
    assert _lib.read_status() == 0


@pytest.mark.parametrize("Sq,Sk,off,causal", [(256, 512, 256, True), (128, 640, 256, True), (256, 384, 0, False), (384, 384, 0, True)])
def test_flash_attention_rectangular_fwd_bwd(Sq, Sk, off, causal):
    from mindformers_b200.ops import attention as A
    torch.manual_seed(Sq + Sk + off)
    B, nq, nkv = 2, 4, 2
    q = (torch.randn(B, Sq, nq, 128, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_()
    k = (torch.randn(B, Sk, nkv, 128, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_()
    v = (torch.randn(B, Sk, nkv, 128, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_()
    o = A.flash_attention_rect(q, k, v, off, causal)
    g = (torch.randn_like(o) * 0.1)
    o.backward(g)
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    ref = Fn.attention_reference(qr, kr, vr, causal, None, q_offset=off)
    ref.backward(g.float())
    assert torch.allclose(o.float(), ref, rtol=3e-2, atol=3e-2)
    for a, b in ((q.grad, qr.grad), (k.grad, kr.grad), (v.grad, vr.grad)):
        assert (a.float() - b).norm() / (b.norm() + 1e-9) < 3e-2
    assert _lib.read_status() == 0


@pytest.mark.parametrize("hd,nq,nkv,block", [(128, 32, 8, 128), (128, 8, 8, 16), (64, 16, 2, 32), (128, 16, 1, 64)])
def test_paged_decode_attention_split_kv(hd, nq, nkv, block):
    torch.manual_seed(hd + nq)
    lib = _lib.get_lib()
    lens = [1, 37, 700, 1300, 64]
    B = len(lens)
    max_blocks = (max(lens) + block - 1) // block + 1
    nblocks = B * max_blocks + 3
    kc = (torch.randn(nblocks, block, nkv, hd, device="cuda") * 0.5).to(torch.bfloat16)
    vc = (torch.randn(nblocks, block, nkv, hd, device="cuda") * 0.5).to(torch.bfloat16)
    perm = torch.randperm(nblocks)[:B * max_blocks].to(torch.int32).view(B, max_blocks).cuda()
    q = (torch.randn(B, nq, hd, device="cuda") * 0.5).to(torch.bfloat16)
    out = torch.empty_like(q)
    ctx = torch.tensor(lens, dtype=torch.int32, device="cuda")
    splits = lib.mfb_paged_decode_splits(B, nkv, block, max_blocks)
    scratch = torch.empty(lib.mfb_paged_decode_scratch_bytes(B, nq, hd, splits) // 4, device="cuda")
    rc = lib.mfb_paged_decode_attention(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), perm.data_ptr(), ctx.data_ptr(), out.data_ptr(),
                                        scratch.data_ptr(), splits, B, nq, nkv, hd, block, max_blocks, hd ** -0.5, _lib.stream_ptr())
    _lib.check(rc, "paged decode")
    for b, n in enumerate(lens):
        rows = perm[b].long()
        kk = kc[rows].reshape(-1, nkv, hd)[:n]
        vv = vc[rows].reshape(-1, nkv, hd)[:n]
        ref = Fn.attention_reference(q[b:b + 1].unsqueeze(0).float(), kk.unsqueeze(0).float(), vv.unsqueeze(0).float(), causal=False)
        assert torch.allclose(out[b].float(), ref[0, 0], rtol=2e-2, atol=2e-2), (b, (out[b].float() - ref[0, 0]).abs().max())


@pytest.mark.parametrize("nq,nkv,block", [(32, 8, 128), (8, 8, 16), (16, 1, 64), (28, 4, 32), (6, 2, 128)])
def test_paged_decode_attention_on_tensor_cores(nq, nkv, block):
    """tcgen05 decode attention over the paged bf16 cache against fp32 attention: ragged lengths (one token, a full
    tile, several tiles + a tail), random block tables with unallocated (-1) tail entries, groups of 1 - 16 query
    heads per KV head, every block size; forced split counts; same bits on a second run."""
    torch.manual_seed(nq * 7 + block)
    lib = _lib.get_lib()
    hd = 128
    assert lib.mfb_paged_decode_tc_supported(nq, nkv, hd, block)
    lens = [1, 37, 128, 700, 1300, 129]
    B = len(lens)
    max_blocks = (max(lens) + block - 1) // block + 2
    nblocks = B * max_blocks + 3
    kc = (torch.randn(nblocks, block, nkv, hd, device="cuda") * 0.5).to(torch.bfloat16)
    vc = (torch.randn(nblocks, block, nkv, hd, device="cuda") * 0.5).to(torch.bfloat16)
    perm = torch.randperm(nblocks)[:B * max_blocks].to(torch.int32).view(B, max_blocks).cuda()
    table = perm.clone()
    for b, n in enumerate(lens):
        table[b, (n + block - 1) // block:] = -1          # blocks that were never allocated
    q = (torch.randn(B, nq, hd, device="cuda") * 0.5).to(torch.bfloat16)
    ctx = torch.tensor(lens, dtype=torch.int32, device="cuda")
    auto = lib.mfb_paged_decode_tc_splits(B, nkv, max_blocks * block)
    outs = []
    for splits in (auto, 1, 3, auto):
        out = torch.full((B + 2, nq, hd), 9.0, device="cuda", dtype=torch.bfloat16)
        scratch = torch.empty(lib.mfb_paged_decode_scratch_bytes(B, nq, hd, splits) // 4, device="cuda")
        rc = lib.mfb_paged_decode_attention_tc(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), table.data_ptr(), ctx.data_ptr(),
                                               out[1:].data_ptr(), scratch.data_ptr(), splits, B, nq, nkv, nblocks, block,
                                               max_blocks, hd ** -0.5, _lib.status_word(q.device).data_ptr(),
                                               _lib.stream_ptr())
        _lib.check(rc, "paged decode tc")
        torch.cuda.synchronize()
        assert _lib.read_status() == 0
        assert torch.all(out[0] == 9.0) and torch.all(out[B + 1] == 9.0)
        outs.append(out[1:B + 1].clone())
        for b, n in enumerate(lens):
            rows = perm[b].long()
            kk = kc[rows].reshape(-1, nkv, hd)[:n]
            vv = vc[rows].reshape(-1, nkv, hd)[:n]
            ref = Fn.attention_reference(q[b:b + 1].unsqueeze(0).float(), kk.unsqueeze(0).float(), vv.unsqueeze(0).float(),
                                         causal=False)
            err = (outs[-1][b].float() - ref[0, 0]).abs().max().item()
            assert err < 2e-2, (splits, b, err)
    assert torch.equal(outs[0], outs[3])


@pytest.mark.parametrize("B,S,nh,causal", [(1, 128, 2, True), (2, 512, 4, True), (1, 1024, 16, True), (1, 384, 3, False)])
def test_flash_attention_mla_shape_forward(B, S, nh, causal):
    """Forward kernel with 192-wide q/k heads and 128-wide v heads against fp32 softmax attention."""
    from mindformers_b200.ops import attention as native
    torch.manual_seed(S + nh)
    q = (torch.randn(B, S, nh, 192, device="cuda") * 0.5).to(torch.bfloat16)
    k = (torch.randn(B, S, nh, 192, device="cuda") * 0.5).to(torch.bfloat16)
    v = (torch.randn(B, S, nh, 128, device="cuda") * 0.5).to(torch.bfloat16)
    assert native.mla_supported(q, k, v)
    scale = 192 ** -0.5
    out = native.mla_forward(q, k, v, causal, scale)
    torch.cuda.synchronize()
    assert _lib.read_status() == 0
    s = torch.einsum("bqhd,bkhd->bhqk", q.float(), k.float()) * scale
    if causal:
        s = s.masked_fill(torch.triu(torch.ones(S, S, device="cuda", dtype=torch.bool), 1), float("-inf"))
    ref = torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s, -1), v.float())
    assert (out.float() - ref).abs().max().item() < 2e-2


@pytest.mark.parametrize("variant", ["single", "cluster"])
@pytest.mark.parametrize("nh,block", [(16, 128), (128, 128), (20, 16), (16, 64)])
def test_mla_decode_attention(nh, block, variant):
    """Absorbed-query MLA decode over the paged latent cache against an fp32 reference, both kernel variants."""
    from mindformers_b200.inference.paged_attention import mla_decode_attention, set_mla_decode_variant
    torch.manual_seed(nh + block)
    default = "cluster" if _lib.get_lib().mfb_mla_decode_get_variant() == 1 else "single"
    set_mla_decode_variant(variant)
    lens = [1, 127, 128, 300, 2304, 129]
    B = len(lens)
    max_blocks = (max(lens) + block - 1) // block + 1
    nblocks = B * max_blocks + 3
    cache = (torch.randn(nblocks, block, 1, 576, device="cuda") * 0.5).to(torch.bfloat16)
    tables = torch.randperm(nblocks)[:B * max_blocks].to(torch.int32).view(B, max_blocks).cuda()
    q = (torch.randn(B, nh, 576, device="cuda") * 0.3).to(torch.bfloat16)
    ctx = torch.tensor(lens, dtype=torch.int32, device="cuda")
    scale = 192 ** -0.5
    try:
        out = mla_decode_attention(q, cache, tables, ctx, block, scale)
        torch.cuda.synchronize()
    finally:
        set_mla_decode_variant(default)
    assert _lib.read_status() == 0
    for b, n in enumerate(lens):
        lat = cache[tables[b].long()].reshape(-1, 576)[:n].float()
        s = (q[b].float() @ lat.t()) * scale
        ref = torch.softmax(s, dim=-1) @ lat[:, :512]
        err = (out[b].float() - ref).abs().max().item()
        assert err < 2e-2, (b, n, err)


@pytest.mark.parametrize("T,N,K", [(128, 128, 128), (300, 512, 1024), (4096, 2048, 7168),
                                   # up to 64 tokens: the kernel with the weight on the MMA rows (32 / 64 token
                                   # columns), K split over a cluster of 8, 4, 2 CTAs or not at all
                                   (64, 1536, 7168), (64, 3072, 1536), (17, 7168, 2048), (1, 256, 512), (33, 24576, 256),
                                   # 65 - 128 tokens: 128-row tiles, K split over a cluster of 8, 2, 4 CTAs
                                   (100, 1536, 7168), (128, 7168, 2048), (128, 4608, 7168)])
def test_fp8_blockscaled_gemm_dense(T, N, K):
    torch.manual_seed(T + N)
    x = (torch.randn(T, K, device="cuda") * 0.7).to(torch.bfloat16)
    w = torch.randn(N, K, device="cuda") * 0.05
    wq, sb = Fn.quantize_weight_128x128(w)
    xq, sa = Fn.quantize_act_1x128(x)
    # the activation quantiser matches the PyTorch one
    xq_ref, sa_ref = Fn.quantize_act_1x128(x.cpu())
    assert torch.allclose(sa[:, :T].cpu(), sa_ref[:, :T], rtol=1e-6)
    assert (xq.float().cpu() - xq_ref.float()).abs().max() <= 32.0   # at most one e4m3 step at the top of the range
    y = Fn.fp8_gemm(xq, sa, wq, sb)
    ref = Fn.fp8_gemm_reference(xq, sa, wq, sb)
    assert (y.float() - ref).norm() / ref.norm() < 5e-3
    full = x.float() @ w.t()
    assert (y.float() - full).norm() / full.norm() < 6e-2     # quantisation error of the format itself
    assert _lib.read_status() == 0


def test_fp8_blockscaled_gemm_grouped():
    torch.manual_seed(9)
    G, N, K = 4, 256, 512
    blocks = [0, 0, 2, 3, 3, 3]            # expert of each 128-row block (expert 1 has no tokens)
    T = len(blocks) * 128
    x = (torch.randn(T, K, device="cuda") * 0.7).to(torch.bfloat16)
    w = torch.randn(G, N, K, device="cuda") * 0.05
    wq, sb = Fn.quantize_weight_128x128(w)
    xq, sa = Fn.quantize_act_1x128(x)
    bg = torch.tensor(blocks + [0, 0], dtype=torch.int32, device="cuda")
    nb = torch.tensor([len(blocks)], dtype=torch.int32, device="cuda")
    xq_pad = torch.cat([xq, torch.zeros(256, K, dtype=xq.dtype, device="cuda")])
    sa_pad = torch.ones(K // 128, T + 256, device="cuda")
    sa_pad[:, :T] = sa[:, :T]
    y = Fn.fp8_gemm(xq_pad, sa_pad, wq, sb, block_group=bg, num_blocks=nb)
    for i, g in enumerate(blocks):
        rows = slice(i * 128, (i + 1) * 128)
        ref = Fn.fp8_gemm_reference(xq[rows], sa[:, rows], wq[g], sb[g])
        assert (y[rows].float() - ref).norm() / ref.norm() < 5e-3, i
    assert _lib.read_status() == 0
    # the same call with the segment fill known: only the rows in use are computed (few-rows-per-expert kernel)
    fill = [200, 0, 3, 290]                # rows in use of every expert: blocks 0-1, -, 2, 3-5
    offs = torch.tensor([0, 256, 256, 384, 768], dtype=torch.int32, device="cuda")
    limit, Fn.FP8_DECODE_MAX_ROWS_PER_GROUP = Fn.FP8_DECODE_MAX_ROWS_PER_GROUP, 1 << 20
    try:
        y2 = Fn.fp8_gemm(xq_pad, sa_pad, wq, sb, block_group=bg, num_blocks=nb, group_offsets=offs,
                         seg_fill=torch.tensor(fill, dtype=torch.int32, device="cuda"))
    finally:
        Fn.FP8_DECODE_MAX_ROWS_PER_GROUP = limit
    for g, n in enumerate(fill):
        if n:
            rows = slice(int(offs[g]), int(offs[g]) + n)
            ref = Fn.fp8_gemm_reference(xq[rows], sa[:, rows], wq[g], sb[g])
            assert (y2[rows].float() - ref).norm() / ref.norm() < 5e-3, g
    assert _lib.read_status() == 0


def test_bounded_peer_wait_reports_status_instead_of_hanging():
    """A cross-rank barrier whose peer never arrives: the kernel gives up after its time limit, records the timeout in
    the status word and returns; the context stays usable."""
    import ctypes
    import time
    lib = _lib.get_lib()
    words = lib.mfb_moe_flag_words()
    mine = torch.zeros(words, dtype=torch.int32, device="cuda")
    absent = torch.zeros(words, dtype=torch.int32, device="cuda")     # stands for a peer that never launches
    flags = (ctypes.c_longlong * 2)(mine.data_ptr(), absent.data_ptr())
    st = _lib.status_word("cuda")
    st.zero_()
    t0 = time.time()
    epoch = torch.zeros(1, dtype=torch.int32, device="cuda")      # the kernel takes epoch + 1 and stores it back
    rc = lib.mfb_moe_barrier(2, 0, epoch.data_ptr(), 1, flags, st.data_ptr(), _lib.stream_ptr())
    assert rc == 0
    torch.cuda.synchronize()
    waited = time.time() - t0
    assert int(st[0].item()) == 4                # kStatusPeerFlagTimeout (word 0; word 1 is the overflow flag)
    assert int(epoch.item()) == 1
    assert 1.0 < waited < 10.0
    st.zero_()
    assert torch.ones(4, device="cuda").sum().item() == 4.0     # the device still answers


@pytest.mark.parametrize("family", ["llama", "deepseek"])
def test_generate_with_cuda_graph_matches_eager(family):
    """The decode step replayed from a CUDA graph yields the same greedy tokens as eager launches."""
    from mindformers_b200.models import AutoModel
    if family == "llama":
        cfg = dict(model_type="llama", num_hidden_layers=2, hidden_size=512, num_attention_heads=4, num_key_value_heads=2,
                   intermediate_size=1024, vocab_size=1024, max_position_embeddings=512, head_dim=128, block_size=16)
    else:
        cfg = dict(model_type="deepseek_v3", num_hidden_layers=3, hidden_size=512, num_attention_heads=4,
                   num_key_value_heads=4, intermediate_size=1024, moe_intermediate_size=256, n_routed_experts=8,
                   n_shared_experts=1, num_experts_per_tok=2, n_group=2, topk_group=1, routed_scaling_factor=1.0,
                   norm_topk_prob=True, scoring_func="sigmoid", first_k_dense_replace=1, vocab_size=1024,
                   q_lora_rank=256, kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128,
                   max_position_embeddings=512, moe_router_enable_expert_bias=True, block_size=128)
    torch.manual_seed(0)
    model = AutoModel.from_config(cfg, device="cuda").eval()
    g = torch.Generator().manual_seed(1)
    prompts = torch.randint(3, 1024, (3, 128), generator=g).tolist()
    eager = model.generate(prompts, max_new_tokens=12, do_sample=False, eos_token_id=None)
    graphed = model.generate(prompts, max_new_tokens=12, do_sample=False, eos_token_id=None, use_cuda_graph=True,
                             device_loop=False)
    assert eager == graphed
    # selection and state update on the device, tokens read back once per burst of 5 steps; the second call replays the
    # graph that the first one captured
    for _ in range(2):
        looped = model.generate(prompts, max_new_tokens=12, do_sample=False, eos_token_id=None, use_cuda_graph=True,
                                device_loop_steps=5)
        assert looped == eager
    stop = eager[1][128 + 4]
    assert model.generate(prompts, max_new_tokens=12, do_sample=False, eos_token_id=stop, use_cuda_graph=True,
                          device_loop_steps=5) == model.generate(prompts, max_new_tokens=12, do_sample=False,
                                                                 eos_token_id=stop)
    entries = list(model._device_loops.values())
    assert len(entries) == 1 and entries[0]["captures"] == 1
    assert _lib.read_status() == 0


def test_decode_advance_kernel_matches_the_reference_and_samples_the_softmax():
    from mindformers_b200.generation.device_loop import DecodeState, decode_advance
    torch.manual_seed(3)
    B, V, width, bs, cap = 37, 32003, 9, 16, 4

    def fresh(device):
        st = DecodeState.allocate(B, width, bs, cap, device)
        g = torch.Generator().manual_seed(1)
        table = torch.randint(0, 500, (B, width), generator=g, dtype=torch.int32)
        table[5, 3:] = -1
        pos = torch.randint(0, width * bs - 2, (B,), generator=g)
        pos[7] = width * bs - 1                       # the next position is outside the table
        fin = [i % 11 == 0 for i in range(B)]
        lim = [int(p) + (2 if i % 5 == 0 else 40) for i, p in enumerate(pos)]
        st.load(list(range(B)), pos.tolist(), table.numpy(), [0] * B, fin, lim)
        st.set_sampling([17, 4242], 0.0, 0)
        return st
    logits = torch.randn(B, V + 5).to(torch.bfloat16).float()      # bf16-rounded values: ties at the maximum do occur
    logits[3, 17] = 50.0
    logits[9, 4242] = 50.0
    logits[12, 100] = logits[12, 30000] = 60.0                      # a tie: the lower index wins
    cpu, dev = fresh("cpu"), fresh("cuda")
    for _ in range(3):
        decode_advance(logits[:, :V], cpu)
        decode_advance(logits.cuda()[:, :V], dev)
    torch.cuda.synchronize()
    for name in ("tok", "pos", "lens", "slots", "hist", "count", "finished"):
        assert torch.equal(getattr(cpu, name), getattr(dev, name).cpu()), name
    assert dev.hist[12, 0].item() == 100 and dev.finished[3].item() == 1 and dev.finished[7].item() == 1
    # sampling: 4096 rows with the same logits, one draw each
    n = 4096
    st = DecodeState.allocate(n, 4, 16, 2, "cuda")
    st.limit.fill_(60)
    st.set_sampling((), 0.5, seed=11)
    row = torch.tensor([2.0, 1.0, 0.0, -1.0, -30.0], device="cuda")
    decode_advance(row[None].repeat(n, 1), st)
    first = st.hist[:, 0].clone()
    freq = torch.bincount(first, minlength=5).float().cpu() / n
    assert (freq - torch.softmax(row.cpu() / 0.5, -1)).abs().max() < 0.03
    st.count.zero_()
    st.pos.zero_()
    decode_advance(row[None].repeat(n, 1), st)
    assert torch.equal(st.hist[:, 0], first)                        # same seed, same history index: same draws
    st.count.zero_()
    st.set_sampling((), 0.5, seed=12)
    decode_advance(row[None].repeat(n, 1), st)
    assert not torch.equal(st.hist[:, 0], first)


@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (300, 1024, 4096), (2048, 6144, 4096), (64, 520, 208), (4096, 4096, 14336)])
def test_w8a8_gemm_matches_exact_integer_product(M, N, K):
    """int8 x int8 on the integer tensor-core path with an int32 accumulator: the result is the exactly computed integer
    product times the scales (plus bias), rounded to bf16 once; ragged M, N and K tails included."""
    torch.manual_seed(M + N)
    a = torch.randint(-127, 128, (M, K), device="cuda", dtype=torch.int8)
    b = torch.randint(-127, 128, (N, K), device="cuda", dtype=torch.int8)
    sa = torch.rand(M, device="cuda") * 0.02 + 0.001
    sb = torch.rand(N, device="cuda") * 0.02 + 0.001
    bias = torch.randn(N, device="cuda").to(torch.bfloat16)
    for use_bias in (False, True):
        y = Fn.w8a8_gemm(a, sa, b, sb, bias if use_bias else None)
        torch.cuda.synchronize()
        assert _lib.read_status() == 0
        acc = (a.double() @ b.double().t())                              # exact: |sum| < 2^53
        ref = acc * sa.double()[:, None] * sb.double()[None, :]
        if use_bias:
            ref = ref + bias.double()
        err = (y.double() - ref).abs().max().item()
        assert err <= ref.abs().max().item() * 2 ** -8 + 1e-6, err        # one bf16 rounding


def test_quantize_act_int8_and_w8a8_linear_against_fp32():
    torch.manual_seed(77)
    x = (torch.randn(1000, 4096, device="cuda") * 2).to(torch.bfloat16)
    w = torch.randn(1024, 4096, device="cuda") * 0.05
    smooth = torch.rand(4096, device="cuda") + 0.5
    for sm in (None, smooth):
        xq, xs = Fn.quantize_act_int8(x, sm)
        xf = x.float() / sm if sm is not None else x.float()
        amax = xf.abs().amax(-1)
        assert torch.allclose(xs, amax / 127.0, rtol=1e-6)
        ref_q = torch.round(xf / xs[:, None]).clamp(-127, 127)
        assert (xq.float() - ref_q).abs().max().item() <= 1                # ties may round either way
        assert ((xq.float() - ref_q).abs() > 0).float().mean().item() < 1e-3
    from mindformers_b200.modules import quantizers as Q
    wq, ws = Q.quantize_weight_rtn(w, "int8", 0)
    y = Fn.w8a8_linear(x, wq, ws[:, 0])
    ref = x.float() @ w.t()
    assert ((y.float() - ref).norm() / ref.norm()).item() < 0.02


@pytest.mark.parametrize("hd,nq,nkv,block", [(128, 32, 8, 16), (64, 8, 2, 128), (128, 4, 4, 32)])
def test_int8_kv_cache_write_decode_and_gather(hd, nq, nkv, block):
    """Keys and values go into the int8 paged cache through the quantising write kernel; the decode kernel and the
    de-quantising gather read them back. Reference: fp32 attention over the de-quantised cache contents."""
    from mindformers_b200.inference.paged_attention import KVCacheContext, _write_cache
    torch.manual_seed(hd + nq)
    lib = _lib.get_lib()
    lens = [1, 37, 700, 1300, 64]
    B = len(lens)
    max_blocks = (max(lens) + block - 1) // block + 1
    nblocks = B * max_blocks + 3
    cache = KVCacheContext(1, nblocks, block, nkv, hd, torch.bfloat16, "cuda", kv_cache_dtype="int8")
    perm = torch.randperm(nblocks)[:B * max_blocks].to(torch.int32).view(B, max_blocks).cuda()
    ks, vs, slots = [], [], []
    for b, n in enumerate(lens):
        ks.append((torch.randn(n, nkv, hd, device="cuda") * (0.2 + b)).to(torch.bfloat16))
        vs.append((torch.randn(n, nkv, hd, device="cuda") * 0.5).to(torch.bfloat16))
        t = torch.arange(n, device="cuda")
        slots.append(perm[b].long()[t // block] * block + t % block)
    k_all, v_all = torch.cat(ks), torch.cat(vs)
    cache.slot_mapping = torch.cat(slots).to(torch.int32)
    _write_cache(cache, 0, k_all, v_all)
    torch.cuda.synchronize()
    kc, vc = cache.key_cache[0], cache.value_cache[0]
    sl = cache.slot_mapping.long()
    kd = kc.view(-1, nkv, hd)[sl].float() * cache.key_scale[0].view(-1, nkv)[sl].unsqueeze(-1)
    vd = vc.view(-1, nkv, hd)[sl].float() * cache.value_scale[0].view(-1, nkv)[sl].unsqueeze(-1)
    # the stored codes reproduce the inputs to within half a quantisation step
    step = k_all.float().abs().amax(-1, keepdim=True) / 127.0
    assert ((kd - k_all.float()).abs() <= 0.51 * step + 1e-6).all()
    assert int(kc.view(-1, nkv, hd)[sl].abs().max()) == 127
    q = (torch.randn(B, nq, hd, device="cuda") * 0.5).to(torch.bfloat16)
    out = torch.empty_like(q)
    ctx = torch.tensor(lens, dtype=torch.int32, device="cuda")
    splits = lib.mfb_paged_decode_splits(B, nkv, block, max_blocks)
    scratch = torch.empty(lib.mfb_paged_decode_scratch_bytes(B, nq, hd, splits) // 4, device="cuda")
    rc = lib.mfb_paged_decode_attention_ex(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), cache.key_scale[0].data_ptr(),
                                           cache.value_scale[0].data_ptr(), perm.data_ptr(), ctx.data_ptr(), out.data_ptr(),
                                           scratch.data_ptr(), splits, B, nq, nkv, hd, block, max_blocks, hd ** -0.5,
                                           _lib.stream_ptr())
    _lib.check(rc, "paged decode int8")
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device="cuda")
    gathered = torch.empty(sum(lens), nkv, hd, device="cuda", dtype=torch.bfloat16)
    rc = lib.mfb_gather_cache_int8(kc.data_ptr(), cache.key_scale[0].data_ptr(), perm.data_ptr(), cu.data_ptr(),
                                   gathered.data_ptr(), B, max(lens), block, max_blocks, nkv, hd, _lib.stream_ptr())
    _lib.check(rc, "gather int8")
    torch.cuda.synchronize()
    assert torch.allclose(gathered.float(), kd.to(torch.bfloat16).float())
    o = 0
    for b, n in enumerate(lens):
        ref = Fn.attention_reference(q[b:b + 1].unsqueeze(0).float(), kd[o:o + n].unsqueeze(0), vd[o:o + n].unsqueeze(0),
                                     causal=False)
        assert torch.allclose(out[b].float(), ref[0, 0], rtol=2e-2, atol=2e-2), (b, (out[b].float() - ref[0, 0]).abs().max())
        o += n


@pytest.mark.parametrize("T", [1, 7, 16, 17, 32, 33, 64])
@pytest.mark.parametrize("N,K", [(6144, 4096), (4096, 14336), (1000, 520), (28672, 1024), (256, 64), (20000, 2048)])
def test_bf16_decode_gemm_matches_fp32_reference(T, N, K):
    """Weight-on-rows product for 1 - 64 rows of activations: every K split (cluster reduce-scatter through distributed
    shared memory), the two-CTAs-per-SM variant and the launcher's own choice, ragged N and K included; canary rows
    around the output stay untouched."""
    torch.manual_seed(T * 131 + N)
    x = (torch.randn(T, K, device="cuda") * 0.5).to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
    ref = x.float() @ w.float().t()
    tol = 2e-2 * ref.abs().max().item() + 1e-3
    try:
        for ks in (0, 1, 2, 4, 8, 16):
            Fn.set_decode_gemm(True, ks)
            buf = torch.full((T + 2, N), 7.0, device="cuda", dtype=torch.bfloat16)
            y = Fn.gemm(x, w, out=buf[1:T + 1])
            torch.cuda.synchronize()
            assert _lib.read_status() == 0
            assert (y.float() - ref).abs().max().item() < tol, (ks, (y.float() - ref).abs().max().item())
            assert torch.all(buf[0] == 7.0) and torch.all(buf[T + 1] == 7.0)
            again = Fn.gemm(x, w)
            assert torch.equal(again, y)                       # same bits on every run (fixed summation order)
            bias = (torch.randn(N, device="cuda") * 0.5).to(torch.bfloat16)
            with torch.no_grad():
                yb = Fn.linear(x, w, bias)                     # bias in the kernel's epilogue
            assert (yb.float() - (ref + bias.float())).abs().max().item() < tol + 4e-3 * bias.abs().max().item()
            assert (yb.float() - y.float() - bias.float()).abs().max().item() <= 2 ** -7 * (ref.abs().max().item() + 2.0)
    finally:
        Fn.set_decode_gemm(True, 0)
