"""Numerics of every hand-written CUDA kernel against a plain PyTorch fp32 statement of the op."""
import math

import pytest
import torch

from oneflow_b200.ops import gemm as G
from oneflow_b200.ops import kernels as K
from oneflow_b200.ops import _native

pytestmark = pytest.mark.gpu
DEV = "cuda"
BF = torch.bfloat16


def close(a, b, rtol=1e-2, atol=None):
    """Element-wise bound ``|a - b| <= atol + rtol * |b|`` against the fp32 statement. ``rtol`` covers the rounding of a
    bf16 result (2^-8) with margin; ``atol`` defaults to 1 % of the reference's RMS, which is what cancellation in an
    fp32-accumulated sum of bf16 products can leave on elements that are themselves close to zero."""
    a, b = a.float().cpu(), b.float().cpu()
    assert a.shape == b.shape, (a.shape, b.shape)
    if atol is None:
        atol = 1e-2 * float(b.pow(2).mean().sqrt()) + 1e-6
    bad = (a - b).abs() > atol + rtol * b.abs()
    if bad.any():
        idx = torch.nonzero(bad)[0].tolist()
        raise AssertionError(f"{int(bad.sum())} of {bad.numel()} elements outside atol={atol:.3g} rtol={rtol}: first at {idx}, "
                             f"got {a[tuple(idx)].item()}, expected {b[tuple(idx)].item()}, max err {(a - b).abs().max().item()}")


@pytest.fixture(autouse=True)
def _status_clean():
    yield
    torch.cuda.synchronize()
    assert _native.read_status() == (0, 0)


@pytest.mark.parametrize("al,bl", [("mk", "nk"), ("mk", "kn"), ("km", "nk"), ("km", "kn")])
@pytest.mark.parametrize("shape", [(128, 128, 64), (520, 392, 264), (2048, 1024, 512)])
def test_gemm_layouts(al, bl, shape):
    M, N, K_ = shape
    torch.manual_seed(1)
    a = torch.randn((M, K_) if al == "mk" else (K_, M), device=DEV, dtype=BF)
    b = torch.randn((N, K_) if bl == "nk" else (K_, N), device=DEV, dtype=BF)
    out = G.gemm(a, b, a_layout=al, b_layout=bl)
    ref = G.gemm_reference(a.cpu(), b.cpu(), al, bl)
    close(out, ref)


@pytest.mark.parametrize("al,bl", [("mk", "nk"), ("mk", "kn"), ("km", "nk"), ("km", "kn")])
@pytest.mark.parametrize("shape", [(512, 768, 320), (1031, 520, 264), (256, 256, 64)])
def test_gemm_two_sm_kernel_layouts(al, bl, shape):
    """The cta_group::2 kernel (256 x 256 tiles over a CTA pair), forced with bn=512 on small and ragged problems."""
    M, N, K_ = shape
    torch.manual_seed(5)
    a = torch.randn((M, K_) if al == "mk" else (K_, M + (-M) % 8), device=DEV, dtype=BF)
    if al == "km":
        a = a[:, :M] if a.shape[1] != M else a
    b = torch.randn((N, K_) if bl == "nk" else (K_, N), device=DEV, dtype=BF)
    out = G.gemm(a, b, a_layout=al, b_layout=bl, bn=512)
    close(out, G.gemm_reference(a.cpu(), b.cpu(), al, bl))


@pytest.mark.parametrize("shape", [(512, 768, 320), (1031, 520, 264)])
def test_gemm_two_sm_kernel_epilogues(shape):
    M, N, K_ = shape
    torch.manual_seed(6)
    a = torch.randn(M, K_, device=DEV, dtype=BF)
    b = torch.randn(N, K_, device=DEV, dtype=BF)
    bias = torch.randn(N, device=DEV, dtype=BF)
    res = torch.randn(M, N, device=DEV, dtype=BF)
    for act in (0, 1, 2, 3):
        out, aux = G.gemm(a, b, bias=bias, act=act, residual=res, want_aux=True, bn=512)
        ref, raux = G.gemm_reference(a.cpu(), b.cpu(), bias=bias.cpu(), act=act, residual=res.cpu(), want_aux=True)
        close(out, ref)
        close(aux, raux)
        if act:
            out = G.gemm(a, b, aux_in=res, act=act, bn=512)
            close(out, G.gemm_reference(a.cpu(), b.cpu(), aux_in=res.cpu(), act=act))
    acc = torch.randn(M, N, device=DEV, dtype=torch.float32)
    ref = G.gemm_reference(a.cpu(), b.cpu(), out=acc.cpu().clone(), accumulate=True, out_dtype=torch.float32, alpha=0.5)
    close(G.gemm(a, b, out=acc, accumulate=True, alpha=0.5, bn=512), ref)
    out32 = G.gemm(a, b, out_dtype=torch.float32, bn=512)
    close(out32, G.gemm_reference(a.cpu(), b.cpu(), out_dtype=torch.float32), rtol=1e-3)


def test_gemm_default_dispatch_reaches_two_sm_kernel():
    """A problem large enough for the dispatcher's own choice of the two-SM kernel (>= 74 tiles of 256 x 256)."""
    torch.manual_seed(7)
    M, N, K_ = 2560, 2048, 256
    a = torch.randn(M, K_, device=DEV, dtype=BF)
    b = torch.randn(N, K_, device=DEV, dtype=BF)
    bias = torch.randn(N, device=DEV, dtype=BF)
    out = G.gemm(a, b, bias=bias, act=2)
    close(out, G.gemm_reference(a.cpu(), b.cpu(), bias=bias.cpu(), act=2))


@pytest.mark.parametrize("kind,code", [(0, 1), (1, 2), (2, 2)])
def test_bounded_wait_runs_out_and_context_stays_usable(kind, code):
    """Every device-side wait of the library has a limit. Here a one-block kernel waits 5 ms for something that never
    happens (kind 0: an mbarrier nobody arrives on; 1: a peer flag nobody writes; 2: a counter nobody advances): it must
    return by itself, leave the matching status code (1 = mbarrier time-out, 2 = peer time-out), and the next kernel
    must run normally."""
    import ctypes
    from ctypes import c_int, c_longlong, c_void_p
    lib = _native.kernels()
    torch.cuda.synchronize()
    assert _native.read_status() == (0, 0)
    elapsed = torch.zeros(1, dtype=torch.int32, device=DEV)
    rc = lib.ofb_wait_probe(c_int(kind), c_longlong(5_000_000), c_void_p(elapsed.data_ptr()), _native.stream_ptr())
    assert rc == 0
    torch.cuda.synchronize()
    st = _native.read_status()          # reads and clears
    assert st[0] == code and st[1] == 7001 + kind, st
    us = int(elapsed.item())
    assert 4_000 <= us <= 500_000, us   # gave up after the limit, not before, and nowhere near the default of seconds
    # the context is intact: a GEMM right after it computes the right thing and the status stays clean
    a = torch.randn(256, 128, device=DEV, dtype=BF)
    b = torch.randn(128, 128, device=DEV, dtype=BF)
    close(G.gemm(a, b), G.gemm_reference(a.cpu(), b.cpu()))
    torch.cuda.synchronize()
    assert _native.read_status() == (0, 0)


@pytest.mark.parametrize("bn", [128, 256])
def test_gemm_epilogues(bn):
    torch.manual_seed(2)
    M, N, K_ = 384, 512, 256
    a = torch.randn(M, K_, device=DEV, dtype=BF)
    b = torch.randn(N, K_, device=DEV, dtype=BF)
    bias = torch.randn(N, device=DEV, dtype=BF)
    res = torch.randn(M, N, device=DEV, dtype=BF)
    for act in (1, 2, 3):
        out, aux = G.gemm(a, b, bias=bias, act=act, residual=res, want_aux=True, bn=bn)
        ref, raux = G.gemm_reference(a.cpu(), b.cpu(), bias=bias.cpu(), act=act, residual=res.cpu(), want_aux=True)
        close(out, ref)
        close(aux, raux)
        out = G.gemm(a, b, aux_in=res, act=act, bn=bn)
        close(out, G.gemm_reference(a.cpu(), b.cpu(), aux_in=res.cpu(), act=act))
    acc = torch.randn(M, N, device=DEV, dtype=torch.float32)
    ref = G.gemm_reference(a.cpu(), b.cpu(), out=acc.cpu().clone(), accumulate=True, out_dtype=torch.float32, alpha=0.5)
    out = G.gemm(a, b, out=acc, accumulate=True, alpha=0.5, bn=bn)
    close(out, ref)


@pytest.mark.parametrize("cols", [64, 1024, 4096, 8192])
def test_layer_norm(cols):
    torch.manual_seed(3)
    rows = 515
    x = torch.randn(rows, cols, device=DEV, dtype=BF) * 2 + 0.5
    g = torch.randn(cols, device=DEV, dtype=BF)
    b = torch.randn(cols, device=DEV, dtype=BF)
    y, mean, rstd = K.layer_norm_fwd(x, g, b, 1e-5)
    ry, rmean, rrstd = K.layer_norm_fwd(x.cpu(), g.cpu(), b.cpu(), 1e-5)
    close(y, ry)
    close(mean, rmean, 1e-3, 1e-3)
    close(rstd, rrstd, 1e-3, 1e-3)
    ref = torch.nn.functional.layer_norm(x.float().cpu(), (cols,), g.float().cpu(), b.float().cpu(), 1e-5)
    close(y, ref)
    dy = torch.randn(rows, cols, device=DEV, dtype=BF)
    add = torch.randn(rows, cols, device=DEV, dtype=BF)
    dx, dg, db = K.layer_norm_bwd(dy, x, g, mean, rstd, add_to_dx=add)
    rdx, rdg, rdb = K.layer_norm_bwd(dy.cpu(), x.cpu(), g.cpu(), rmean, rrstd, add_to_dx=add.cpu())
    close(dx, rdx)
    close(dg, rdg, 2e-2, 5e-2)
    close(db, rdb, 2e-2, 5e-2)


@pytest.mark.parametrize("act", [1, 2, 3])
def test_bias_act(act):
    torch.manual_seed(4)
    x = torch.randn(300, 1024, device=DEV, dtype=BF)
    b = torch.randn(1024, device=DEV, dtype=BF)
    dy = torch.randn(300, 1024, device=DEV, dtype=BF)
    close(K.bias_act_fwd(x, b, act), K.bias_act_fwd(x.cpu(), b.cpu(), act))
    close(K.bias_act_bwd(x, b, dy, act), K.bias_act_bwd(x.cpu(), b.cpu(), dy.cpu(), act))


def test_bias_mask_scale_and_dropout_mask():
    torch.manual_seed(5)
    x = torch.randn(257, 512, device=DEV, dtype=BF)
    b = torch.randn(512, device=DEV, dtype=BF)
    add = torch.randn(257, 512, device=DEV, dtype=BF)
    mask = K.dropout_mask(x.shape, 0.1, seed=1234, device=DEV)
    keep = mask.float().mean().item()
    assert abs(keep - 0.9) < 0.01
    mask2 = K.dropout_mask(x.shape, 0.1, seed=1234, device=DEV)
    assert torch.equal(mask, mask2)
    y = K.bias_mask_scale(x, b, mask, 1 / 0.9, add)
    close(y, K.bias_mask_scale(x.cpu(), b.cpu(), mask.cpu(), 1 / 0.9, add.cpu()))


def test_cast_scale_column_sum():
    torch.manual_seed(6)
    x = torch.randn(1000, 776, device=DEV, dtype=BF)
    st = torch.tensor([0.25], device=DEV)
    y = K.cast_scale(x, 2.0, torch.float32, st)
    close(y, x.float().cpu() * 0.5, 1e-3, 1e-3)
    close(K.column_sum(x), x.float().cpu().sum(0), 1e-2, 1e-2)


@pytest.mark.parametrize("cols", [128, 512, 2048])
def test_softmax_tril(cols):
    torch.manual_seed(7)
    x = torch.randn(2, 3, cols, cols, device=DEV, dtype=BF)
    mask = K.dropout_mask(x.shape, 0.1, seed=7, device=DEV)
    y, sm = K.softmax_fwd(x, scale=0.125, tril=True, dropout_mask=mask, dropout_scale=1 / 0.9, want_softmax=True)
    ry, rsm = K.softmax_fwd(x.cpu(), scale=0.125, tril=True, dropout_mask=mask.cpu(), dropout_scale=1 / 0.9,
                            want_softmax=True)
    close(y, ry)
    close(sm, rsm)
    dy = torch.randn_like(x)
    dx = K.softmax_bwd(sm, dy, scale=0.125, tril=True, dropout_mask=mask, dropout_scale=1 / 0.9)
    rdx = K.softmax_bwd(rsm, dy.cpu(), scale=0.125, tril=True, dropout_mask=mask.cpu(), dropout_scale=1 / 0.9)
    close(dx, rdx, 2e-2, 1e-3)


def test_softmax_attn_mask():
    torch.manual_seed(8)
    B, H, S = 2, 4, 256
    x = torch.randn(B, H, S, S, device=DEV, dtype=BF)
    am = (torch.rand(S, S, device=DEV) > 0.2)
    y = K.softmax_fwd(x, scale=0.5, attn_mask=am)
    ry = K.softmax_fwd(x.cpu(), scale=0.5, attn_mask=am.cpu())
    close(y, ry)


@pytest.mark.parametrize("vocab", [1024, 50304])
def test_xent(vocab):
    torch.manual_seed(9)
    rows = 300
    logits = torch.randn(rows, vocab, device=DEV, dtype=BF) * 3
    labels = torch.randint(0, vocab, (rows,), device=DEV)
    labels[5] = -100
    st = K.xent_stats(logits, labels)
    loss, d = K.xent_grad(logits, labels, st, grad_scale=0.5)
    ref = torch.nn.functional.cross_entropy(logits.float().cpu(), labels.cpu(), reduction="none", ignore_index=-100)
    close(loss, ref, 1e-3, 1e-3)
    lf = logits.float().cpu().requires_grad_(True)
    torch.nn.functional.cross_entropy(lf, labels.cpu(), reduction="sum", ignore_index=-100).mul(0.5).backward()
    close(d, lf.grad, 2e-2, 1e-3)
    # vocabulary-sharded path: two shards merged
    half = vocab // 2
    p0 = K.xent_stats(logits[:, :half].contiguous(), labels, 0)
    p1 = K.xent_stats(logits[:, half:].contiguous(), labels, half)
    merged = K.xent_merge(torch.stack([p0, p1]))
    close(merged[:, 2], st[:, 2], 1e-3, 1e-3)
    l2, _ = K.xent_grad(logits[:, half:].contiguous(), labels, merged, vocab_start=half)
    close(l2, ref, 1e-3, 1e-3)


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("causal", [False, True])
def test_fmha_fwd(D, causal):
    torch.manual_seed(10)
    B, S, H = 2, 384, 3
    qkv = torch.randn(B, S, 3, H, D, device=DEV, dtype=BF)
    q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
    out, lse = K.fmha_fwd(q, k, v, causal=causal)
    ro, rl = K.fmha_reference(q.cpu(), k.cpu(), v.cpu(), causal, 1 / math.sqrt(D))
    close(out, ro)
    close(lse, rl, 1e-2, 1e-2)


def test_fmha_fwd_padding_and_ragged():
    torch.manual_seed(11)
    B, S, H, D = 3, 200, 2, 64
    q = torch.randn(B, S, H, D, device=DEV, dtype=BF)
    k = torch.randn(B, S, H, D, device=DEV, dtype=BF)
    v = torch.randn(B, S, H, D, device=DEV, dtype=BF)
    kv_len = torch.tensor([200, 77, 130], dtype=torch.int32)
    out, lse = K.fmha_fwd(q, k, v, causal=False, kv_len=kv_len)
    ro, rl = K.fmha_reference(q.cpu(), k.cpu(), v.cpu(), False, 1 / math.sqrt(D), kv_len)
    close(out, ro)
    close(lse, rl, 1e-2, 1e-2)


def test_multi_tensor_adamw_sgd_and_norm():
    torch.manual_seed(12)
    sizes = [1000, 65536 + 8, 300000, 16]
    def mk(dt=torch.float32):
        return [torch.randn(n, device=DEV, dtype=dt) for n in sizes]
    w, g, m, v = mk(), mk(BF), [t.abs() * 0 for t in mk()], [t.abs() * 0 for t in mk()]
    c = [torch.empty(n, device=DEV, dtype=BF) for n in sizes]
    wc, gc, mc, vc = [[t.cpu().clone() for t in L] for L in (w, g, m, v)]
    cc = [t.cpu().clone() for t in c]
    kw = dict(lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, scale=0.5, step=3)
    K.multi_tensor_adamw(g, w, c, m, v, **kw)
    K.multi_tensor_adamw(gc, wc, cc, mc, vc, **kw)
    for a, b in zip(w + m + v, wc + mc + vc):
        close(a, b, 1e-3, 1e-4)
    for a, b in zip(c, cc):  # bf16 copies: one rounding step apart at most
        close(a, b, 1e-2, 1e-2)
    # SGD momentum
    w, g, m = mk(), mk(), [t * 0 for t in mk()]
    wc, gc, mc = [[t.cpu().clone() for t in L] for L in (w, g, m)]
    kw = dict(lr=0.1, momentum=0.9, nesterov=True, weight_decay=1e-4, l2=1e-3, scale=2.0)
    K.multi_tensor_sgd(g, w, None, m, **kw)
    K.multi_tensor_sgd(gc, wc, None, mc, **kw)
    for a, b in zip(w + m, wc + mc):
        close(a, b, 1e-3, 1e-4)
    g[1][7] = float("inf")
    out = K.multi_tensor_sqsum(g)
    ref = K.multi_tensor_sqsum([t.cpu() for t in g])
    close(out[:1], ref[:1], 1e-3, 1e-3)
    assert int(out[1].item()) == 1
    f, found, norm = K.clip_factor(out, 1.0)
    assert int(found.item()) == 1 and f.item() <= 1.0


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("causal", [False, True])
def test_fmha_bwd(D, causal):
    torch.manual_seed(13)
    B, S, H = 2, 384, 2
    qkv = torch.randn(B, S, 3, H, D, device=DEV, dtype=BF)
    q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
    out, lse = K.fmha_fwd(q, k, v, causal=causal)
    d_o = torch.randn_like(out)
    dq, dk, dv = K.fmha_bwd(q, k, v, out, d_o, lse, causal=causal)
    rq, rk, rv = K.fmha_bwd_reference(q.cpu(), k.cpu(), v.cpu(), out.cpu(), d_o.cpu(), lse.cpu(), causal,
                                      1 / math.sqrt(D))
    close(dq, rq, 3e-2, 2e-2)
    close(dk, rk, 3e-2, 2e-2)
    close(dv, rv, 3e-2, 2e-2)


def test_fmha_bwd_padding_ragged():
    torch.manual_seed(14)
    B, S, H, D = 2, 200, 2, 64
    qkv = torch.randn(B, S, 3, H, D, device=DEV, dtype=BF)
    q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
    kv_len = torch.tensor([200, 90], dtype=torch.int32)
    out, lse = K.fmha_fwd(q, k, v, causal=False, kv_len=kv_len)
    d_o = torch.randn_like(out)
    dq, dk, dv = K.fmha_bwd(q, k, v, out, d_o, lse, causal=False, kv_len=kv_len)
    rq, rk, rv = K.fmha_bwd_reference(q.cpu(), k.cpu(), v.cpu(), out.cpu(), d_o.cpu(), lse.cpu(), False,
                                      1 / math.sqrt(D), kv_len)
    close(dq, rq, 3e-2, 2e-2)
    close(dk, rk, 3e-2, 2e-2)
    close(dv, rv, 3e-2, 2e-2)


@pytest.mark.parametrize("D,causal,Sq,Sk,H,Hk", [(64, True, 200, 456, 4, 2), (128, True, 384, 256, 4, 1), (64, False, 130, 300, 6, 3),
                                                 (128, True, 256, 256, 8, 2), (64, True, 300, 100, 2, 2)])
def test_fmha_grouped_heads_and_unequal_lengths(D, causal, Sq, Sk, H, Hk):
    """Grouped-query heads (H query heads on Hk key/value heads) and Sq != Sk with the causal diagonal at the bottom-right
    corner (Sq > Sk leaves the first rows without any visible key: zero output, zero gradient), forward and backward."""
    torch.manual_seed(21)
    B = 2
    q = torch.randn(B, Sq, H, D, device=DEV, dtype=BF)
    kv = torch.randn(B, Sk, 2, Hk, D, device=DEV, dtype=BF)
    k, v = kv[:, :, 0], kv[:, :, 1]
    sc = 1 / math.sqrt(D)
    out, lse = K.fmha_fwd(q, k, v, causal=causal)
    ro, rl = K.fmha_reference(q.cpu(), k.cpu(), v.cpu(), causal, sc)
    # probabilities are rounded to bf16 (2^-9 relative) before they multiply V ~ N(0, 1): rows that see a handful of keys sum a
    # few terms of magnitude ~0.3 that partly cancel, so the absolute bound is set from that, not from the output's RMS (which
    # the all-zero rows above the shifted diagonal pull down)
    close(out, ro, 1e-2, 5e-3)
    live = torch.isfinite(rl)
    assert torch.equal(torch.isfinite(lse.cpu()), live)
    close(lse.cpu()[live], rl[live], 1e-2, 1e-2)
    d_o = torch.randn_like(out)
    dq, dk, dv = K.fmha_bwd(q, k, v, out, d_o, lse, causal=causal)
    assert dk.shape == (B, Sk, Hk, D) and dq.shape == (B, Sq, H, D)
    rq, rk, rv = K.fmha_bwd_reference(q.cpu(), k.cpu(), v.cpu(), out.cpu(), d_o.cpu(), lse.cpu(), causal, sc)
    close(dq, rq, 3e-2, 2e-2)
    close(dk, rk, 3e-2, 2e-2 * math.sqrt(H // Hk))
    close(dv, rv, 3e-2, 2e-2 * math.sqrt(H // Hk))


@pytest.mark.parametrize("D,causal,p", [(64, True, 0.1), (128, False, 0.3)])
def test_fmha_dropout_follows_its_philox_mask(D, causal, p):
    """The kernels drop probabilities by a Philox stream indexed by position; forward and backward agree with the fp32
    statement that applies the same mask (written out by the mask kernel), the mask keeps about 1 - p of the entries,
    and another offset gives another mask."""
    torch.manual_seed(22)
    B, S, H = 2, 320, 3
    qkv = torch.randn(B, S, 3, H, D, device=DEV, dtype=BF)
    q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
    sc = 1 / math.sqrt(D)
    seed, off = 0x1234567890ABCDEF, 7
    mask = K.fmha_dropout_mask(B, H, S, S, p, seed, off, DEV)
    frac = mask.float().mean().item()
    assert abs(frac - (1 - p)) < 5e-3, frac
    assert not torch.equal(mask, K.fmha_dropout_mask(B, H, S, S, p, seed, off + 1, DEV))
    assert torch.equal(mask, K.fmha_dropout_mask(B, H, S, S, p, seed, off, DEV))
    out, lse = K.fmha_fwd(q, k, v, causal=causal, dropout_p=p, seed=seed, offset=off)
    ro, rl = K.fmha_reference(q.cpu(), k.cpu(), v.cpu(), causal, sc, None, p, mask.cpu())
    close(out, ro)
    close(lse, rl, 1e-2, 1e-2)
    d_o = torch.randn_like(out)
    dq, dk, dv = K.fmha_bwd(q, k, v, out, d_o, lse, causal=causal, dropout_p=p, seed=seed, offset=off)
    rq, rk, rv = K.fmha_bwd_reference(q.cpu(), k.cpu(), v.cpu(), out.cpu(), d_o.cpu(), lse.cpu(), causal, sc, None, p, mask.cpu())
    close(dq, rq, 3e-2, 2e-2)
    close(dk, rk, 3e-2, 2e-2)
    close(dv, rv, 3e-2, 2e-2)


def test_sdpa_entry_point_runs_the_fused_kernels():
    """flow.nn.functional.scaled_dot_product_attention with grouped heads, Sq != Sk and dropout: fused kernels (the launch
    counter moves), gradients flow, eval-mode result equals torch's op on the same inputs."""
    import oneflow_b200 as flow
    torch.manual_seed(23)
    B, H, Hk, Sq, Sk, D = 2, 4, 2, 128, 256, 64
    q = torch.randn(B, H, Sq, D, device=DEV, dtype=BF, requires_grad=True)
    k = torch.randn(B, Hk, Sk, D, device=DEV, dtype=BF, requires_grad=True)
    v = torch.randn(B, Hk, Sk, D, device=DEV, dtype=BF, requires_grad=True)
    n0 = K.launch_count
    y = flow.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True)
    assert K.launch_count > n0
    kk, vv = (t.repeat_interleave(H // Hk, dim=1) for t in (k, v))
    m = torch.ones(Sq, Sk, dtype=torch.bool, device=DEV).tril(Sk - Sq)
    ref = torch.nn.functional.scaled_dot_product_attention(q.float(), kk.float(), vv.float(), attn_mask=m)
    close(y, ref)
    y2 = flow.nn.functional.scaled_dot_product_attention(q, k, v, dropout_p=0.2)
    y2.float().sum().backward()
    assert q.grad is not None and k.grad.shape == k.shape and torch.isfinite(v.grad.float()).all()


@pytest.mark.parametrize("self_inter,T,D", [(False, 26, 128), (True, 26, 128), (False, 7, 64), (False, 31, 32)])
def test_dot_feature_interaction(self_inter, T, D):
    from oneflow_b200.ops.interaction import dot_feature_interaction, dot_feature_interaction_reference
    torch.manual_seed(3)
    B = 517
    dense = (torch.randn(B, D, device="cuda") * 0.5).bfloat16().requires_grad_()
    sparse = (torch.randn(B, T, D, device="cuda") * 0.5).bfloat16().requires_grad_()
    F = T + 1
    npairs = F * (F + 1) // 2 if self_inter else F * (F - 1) // 2
    pad = (-(D + npairs)) % 8 or 8
    n0 = K.launch_count
    out = dot_feature_interaction([dense, sparse], output_concat=dense, self_interaction=self_inter, output_padding=pad)
    assert K.launch_count == n0 + 1, "native interaction kernel did not run"
    d32, s32 = dense.detach().float().requires_grad_(), sparse.detach().float().requires_grad_()
    ref = dot_feature_interaction_reference([d32, s32], output_concat=d32, self_interaction=self_inter, output_padding=pad)
    assert out.shape == ref.shape
    torch.testing.assert_close(out.float(), ref, atol=0.06, rtol=0.02)
    g = (torch.randn_like(ref) * 0.5).bfloat16()
    out.backward(g)
    ref.backward(g.float())
    torch.testing.assert_close(dense.grad.float(), d32.grad, atol=0.15, rtol=0.03)
    torch.testing.assert_close(sparse.grad.float(), s32.grad, atol=0.15, rtol=0.03)


@pytest.mark.parametrize("N,H,W,Cin,Cout,R", [(4, 56, 56, 64, 64, 3), (3, 28, 28, 128, 128, 3), (5, 14, 14, 256, 256, 3),
                                              (6, 7, 7, 512, 512, 3), (2, 19, 13, 64, 128, 3), (2, 16, 16, 64, 64, 5)])
def test_conv_implicit_gemm(N, H, W, Cin, Cout, R):
    from oneflow_b200.ops import conv as C
    torch.manual_seed(0)
    x = torch.randn(N, H, W, Cin, device="cuda").bfloat16()
    w = (torch.randn(Cout, R, R, Cin, device="cuda") / math.sqrt(R * R * Cin)).bfloat16()
    dy = torch.randn(N, H, W, Cout, device="cuda").bfloat16()
    x32 = x.float().requires_grad_()
    w32 = w.float().requires_grad_()
    ref = C._ref_conv(x32, w32)
    ref.backward(dy.float())
    y = C.conv_fprop(x, w)
    torch.testing.assert_close(y.float(), ref.detach(), atol=3e-2, rtol=2e-2)
    dx = C.conv_dgrad(dy, w)
    torch.testing.assert_close(dx.float(), x32.grad, atol=3e-2, rtol=2e-2)
    dw = C.conv_wgrad(x, dy, (R, R))
    scale = w32.grad.abs().max().item()
    assert (dw - w32.grad).abs().max().item() <= 1e-2 * scale + 1e-3
    dw2 = C.conv_wgrad(x, dy, (R, R), out=dw.clone(), accumulate=True)
    assert (dw2 - 2 * w32.grad).abs().max().item() <= 2e-2 * scale + 2e-3
    torch.cuda.synchronize()
    assert _native.read_status() == (0, 0)


def test_flow_conv2d_channels_last_uses_igemm():
    import oneflow_b200 as flow
    torch.manual_seed(0)
    conv = flow.nn.Conv2d(64, 128, 3, padding=1, bias=True).cuda().bfloat16().to(memory_format=torch.channels_last)
    x = torch.randn(4, 64, 20, 20, device="cuda").bfloat16().to(memory_format=torch.channels_last).requires_grad_()
    n0 = K.launch_count
    y = conv(x)
    assert K.launch_count == n0 + 1, "the eligible convolution must run on the implicit-GEMM kernel"
    assert y.shape == (4, 128, 20, 20) and y.is_contiguous(memory_format=torch.channels_last)
    ref = torch.nn.functional.conv2d(x.detach().float(), conv.weight.detach().float(), conv.bias.detach().float(), padding=1)
    torch.testing.assert_close(y.float(), ref, atol=5e-2, rtol=3e-2)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    wr = conv.weight.detach().float().requires_grad_()
    torch.nn.functional.conv2d(xr, wr, None, padding=1).backward(g.float())
    torch.testing.assert_close(x.grad.float(), xr.grad, atol=8e-2, rtol=3e-2)
    assert (conv.weight.grad.float() - wr.grad).abs().max() <= 2e-2 * wr.grad.abs().max() + 1e-2
    # a strided convolution takes the library path and still works
    conv2 = flow.nn.Conv2d(64, 64, 3, stride=2, padding=1).cuda().bfloat16()
    assert conv2(x.detach()).shape == (4, 64, 10, 10)


def test_profiler_reports_native_kernels_with_bandwidth():
    """Inside flow.profiler.profile the native kernel calls appear by name with device time, input shapes and a bandwidth
    (bytes of the operands / device time); ATen ops appear beside them."""
    import oneflow_b200 as flow
    x = torch.randn(4096, 4096, device=DEV, dtype=BF)
    w = torch.randn(4096, 4096, device=DEV, dtype=BF)
    g, b = torch.ones(4096, device=DEV, dtype=BF), torch.zeros(4096, device=DEV, dtype=BF)
    G.gemm(x, w)
    with flow.profiler.profile(record_shapes=True, record_attrs=True, record_bandwidth_for_cuda=True) as prof:
        with flow.profiler.record_function("step"):
            for _ in range(3):
                y = G.gemm(x, w)
            K.layer_norm_fwd(y, g, b)
            torch.relu(y)
    avg = prof.key_averages(group_by_input_shape=True, group_by_attributes=True)
    by = {e.name: e for e in avg}
    assert by["gemm_bf16"].count == 3 and by["layer_norm_fwd"].count == 1 and by["aten::relu"].count == 1 and by["step"].count == 1
    ge = by["gemm_bf16"]
    assert ge.cuda_time > 20 and ge.flops == 3 * 2.0 * 4096 ** 3         # a 4096^3 GEMM takes > 20 us on any B200
    assert ge.input_shapes == "[(4096,4096), (4096,4096), (4096,4096)]" and "act=0" in ge.attributes
    ln = by["layer_norm_fwd"]
    assert ln.bandwidth is not None and 50 < ln.bandwidth < 20000       # GB/s: two 32 MB passes in some tens of microseconds
    assert by["step"].cuda_time_total >= ge.cuda_time_total
    t = avg.table()
    assert "Bandwidth" in t.splitlines()[0] and "GB/s" in t and "gemm_bf16" in t
    # the library is handed out unwrapped again
    assert type(_native.kernels()).__name__ == "CDLL"


def test_remat_on_cuda_matches_unbounded_run():
    """flow.remat.scope on CUDA tensors: eviction really lowers torch's allocated bytes, backward (on autograd's device thread)
    recomputes what it needs, gradients equal the unbounded run."""
    import oneflow_b200 as flow
    torch.manual_seed(3)
    layers = torch.nn.ModuleList([torch.nn.Linear(1024, 1024) for _ in range(8)]).to(DEV)
    x = torch.randn(2048, 1024, device=DEV)

    def run():
        h = x
        for l in layers:
            h = torch.tanh(l(h)) + h
        return h.pow(2).mean()
    ref = run()
    ref.backward()
    g_ref = [p.grad.clone() for p in layers.parameters()]
    for p in layers.parameters():
        p.grad = None
    act = 2048 * 1024 * 4
    torch.cuda.synchronize()
    torch.cuda.reset_peak_memory_stats()
    base = torch.cuda.memory_allocated()
    with flow.remat.scope(budget=10 * act) as r:
        loss = run()
        assert r.stats["forced_eviction_num"] > 0
        assert torch.cuda.memory_allocated() - base <= 11 * act      # 24 activations were produced, at most the budget is held
        loss.backward()
        assert r.stats["recomputation_num"] > 0
    torch.cuda.synchronize()
    assert torch.allclose(loss, ref)
    for a, p in zip(g_ref, layers.parameters()):
        assert torch.allclose(a, p.grad, atol=1e-6, rtol=1e-5)


def test_mlp_unit_folds_the_activation_gradient_into_the_gemm():
    """fused_ops.mlp == linear(gelu(linear(x))) + residual with the same gradients as the fp32 statement; its backward issues one
    kernel less than the two separate linears (the GELU gradient rides in the second layer's data-gradient GEMM)."""
    from oneflow_b200.framework import fused_ops as FO
    torch.manual_seed(31)
    T, H, F_ = 512, 256, 1024
    x = (torch.randn(T, H, device=DEV) * 0.5).to(BF).requires_grad_()
    w1 = (torch.randn(F_, H, device=DEV) * 0.05).to(BF).requires_grad_()
    b1 = (torch.randn(F_, device=DEV) * 0.1).to(BF).requires_grad_()
    w2 = (torch.randn(H, F_, device=DEV) * 0.05).to(BF).requires_grad_()
    b2 = (torch.randn(H, device=DEV) * 0.1).to(BF).requires_grad_()
    res = (torch.randn(T, H, device=DEV) * 0.5).to(BF).requires_grad_()
    gy = torch.randn(T, H, device=DEV).to(BF)

    def run(fused):
        for t in (x, w1, b1, w2, b2, res):
            t.grad = None
        n0 = K.launch_count
        if fused:
            y = FO.mlp(x, w1, b1, w2, b2, act="gelu", residual=res)
        else:
            y = FO.linear(FO.linear(x, w1, b1, act="gelu"), w2, b2, residual=res)
        y.backward(gy)
        return y.detach(), [t.grad.clone() for t in (x, w1, b1, w2, b2, res)], K.launch_count - n0
    y_f, g_f, n_f = run(True)
    y_s, g_s, n_s = run(False)
    assert n_f == n_s - 1, (n_f, n_s)
    xf, w1f, b1f, w2f, b2f, rf = (t.detach().float().requires_grad_() for t in (x, w1, b1, w2, b2, res))
    ref = torch.nn.functional.linear(torch.nn.functional.gelu(torch.nn.functional.linear(xf, w1f, b1f)), w2f, b2f) + rf
    ref.backward(gy.float())
    close(y_f, ref.detach())

    def rms(t):
        return float(t.float().pow(2).mean().sqrt())
    # gradients pass through two bf16 roundings of [T, ffn]-sized intermediates (one in the folded form): elements that nearly
    # cancel carry an absolute error of a few percent of the tensor's RMS
    for got, want in zip(g_f, (xf, w1f, b1f, w2f, b2f, rf)):
        close(got, want.grad, 2e-2, 3e-2 * rms(want.grad))
    for a, b in zip(g_f, g_s):
        close(a, b.float(), 2e-2, 3e-2 * rms(b))


def test_fused_mlp_chain_on_cuda():
    """flow._C.fused_mlp on bf16 CUDA tensors: three linear + ReLU layers, each ReLU gradient folded into the next layer's
    data-gradient GEMM (no separate activation-gradient kernel runs), values and gradients against the fp32 statement."""
    import oneflow_b200 as flow
    torch.manual_seed(32)
    T = 384
    dims = [256, 512, 384, 128]
    x = (torch.randn(T, dims[0], device=DEV) * 0.5).to(BF).requires_grad_()
    ws = [(torch.randn(dims[i + 1], dims[i], device=DEV) * 0.06).to(BF).requires_grad_() for i in range(3)]
    bs = [(torch.randn(dims[i + 1], device=DEV) * 0.1).to(BF).requires_grad_() for i in range(3)]
    gy = torch.randn(T, dims[-1], device=DEV).to(BF)
    n0 = K.launch_count
    y = flow._C.fused_mlp(x, ws, bs, skip_final_activation=True)
    y.backward(gy)
    # 3 forward GEMMs; backward: 3 data-gradient + 3 weight-gradient GEMMs + 3 bias column sums, no activation-gradient kernel
    assert K.launch_count - n0 == 12, K.launch_count - n0
    # fp32 statement that rounds the hidden activations to bf16 where the kernels store them (straight-through for the
    # gradient): ReLU is discontinuous, so a statement with unrounded hidden values switches a few units per token the other
    # way (|pre-activation| below the rounding noise of its inputs) and its gradients then differ by several percent of
    # their RMS on whole rows: measured 10 - 30 % of the elements beyond 3 % of RMS, against none for GELU
    ref_in = [t.detach().float().requires_grad_() for t in [x] + ws + bs]
    h = ref_in[0]
    for i in range(3):
        h = torch.nn.functional.linear(h, ref_in[1 + i], ref_in[4 + i])
        if i < 2:
            h = torch.relu(h)
            h = h + (h.bfloat16().float() - h).detach()
    h.backward(gy.float())
    close(y, h.detach())

    def rms(t):
        return float(t.float().pow(2).mean().sqrt())
    # even so a hidden value can round to the neighbouring bf16 number in the kernel (other summation order), which now and
    # then switches a unit of the next layer: up to 1 % of the elements may sit outside the bound, none far outside
    for got, want in zip([x] + ws + bs, ref_in):
        g, w_ = got.grad.float(), want.grad
        r = rms(w_)
        bad = (g - w_).abs() > 3e-2 * r + 2e-2 * w_.abs()
        assert bad.float().mean().item() < 0.01, bad.float().mean().item()
        assert (g - w_).abs().max().item() < 0.5 * r
    # and the folded form equals the layer-by-layer form bit for bit
    got = [t.grad.clone() for t in [x] + ws + bs]
    for t in [x] + ws + bs:
        t.grad = None
    from oneflow_b200.framework import fused_ops as FO
    h2 = x
    for i in range(3):
        h2 = FO.linear(h2, ws[i], bs[i], act=("relu" if i < 2 else 0))
    h2.backward(gy)
    for a, t in zip(got, [x] + ws + bs):
        assert torch.equal(a, t.grad)
