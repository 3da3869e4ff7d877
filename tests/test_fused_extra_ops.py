"""The long tail of flow._C fused functions against their straightforward statements (CPU)."""
import math

import torch
import torch.nn.functional as F

from oneflow_b200 import _C
import oneflow as flow
import pytest


def test_fused_glu_modes():
    torch.manual_seed(0)
    x, w, b = torch.randn(5, 16), torch.randn(24, 16), torch.randn(24)
    y = _C.fused_glu(x, w, b, activation="silu")
    h, g = (x @ w.t() + b).chunk(2, -1)
    torch.testing.assert_close(y, h * F.silu(g))
    v, c = torch.randn(12, 16), torch.randn(12)
    y2 = _C.fused_glu(x, w[:12], b[:12], v, c, activation="gelu")
    torch.testing.assert_close(y2, (x @ w[:12].t() + b[:12]) * F.gelu(x @ v.t() + c))


def test_norm_family():
    torch.manual_seed(1)
    x, skip, bias, gamma, beta = torch.randn(4, 32), torch.randn(4, 32), torch.randn(32), torch.rand(32), torch.randn(32)
    y = _C.skip_layer_norm(x, gamma=gamma, beta=beta, bias=bias, skip=skip, epsilon=1e-5, alpha=0.5)
    torch.testing.assert_close(y, F.layer_norm(x + bias + 0.5 * skip, (32,), gamma, beta, 1e-5))
    r = _C.rms_norm(x, gamma, (32,), 1e-6)
    torch.testing.assert_close(r, x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-6) * gamma)
    torch.testing.assert_close(_C.rms_layer_norm(x, gamma, 1e-6), r)
    torch.testing.assert_close(_C.skip_rms_norm(x, weight=gamma, skip=skip, alpha=1.0, epsilon=1e-6), _C.rms_norm(x + skip, gamma, (32,), 1e-6))


def test_cross_interaction_weighted_sum_clip():
    torch.manual_seed(2)
    x, x0, w, b = torch.randn(6, 8), torch.randn(6, 8), torch.randn(1, 8), torch.randn(8)
    torch.testing.assert_close(_C.fused_cross_feature_interaction(x, w, x0, b, "vector"), (x @ w.t()) * x0 + b + x)
    W = torch.randn(8, 8)
    torch.testing.assert_close(_C.fused_cross_feature_interaction(x, W, x0, b, "matrix"), (x @ W.t() + b) * x0 + x)
    ts = [torch.randn(3, 4) for _ in range(3)]
    torch.testing.assert_close(_C.fused_weighted_sum(ts, [0.1, 0.2, 0.3], 2.0), 2.0 * (0.1 * ts[0] + 0.2 * ts[1] + 0.3 * ts[2]))
    grads = [torch.randn(10), torch.randn(5, 5)]
    norm = torch.cat([g.flatten() for g in grads]).norm()
    total = _C.fused_clip_grad(grads, 1.0, 2.0)
    torch.testing.assert_close(total, norm)
    assert abs(torch.cat([g.flatten() for g in grads]).norm().item() - 1.0) < 1e-3
    torch.testing.assert_close(_C.fused_fast_gelu_mul(x, x0), F.gelu(x, approximate="tanh") * x0)


def test_attention_helpers_and_rotary():
    torch.manual_seed(3)
    s = torch.randn(2, 3, 5, 5)
    t = _C.fused_scale_tril(s, 0, -1e4, 0.5)
    assert torch.all(t[..., 0, 1:] == -1e4) and torch.allclose(t[..., 2, :3], s[..., 2, :3] * 0.5)
    hs = torch.randn(7, 2, 3 * 4 * 8)
    qk, v = _C.fused_self_attention(hs, head_size=8, alpha=0.25)
    assert qk.shape == (2, 4, 7, 7) and v.shape == (7, 2, 32)
    q = hs.view(7, 2, 4, 3, 8)[..., 0, :]
    k = hs.view(7, 2, 4, 3, 8)[..., 1, :]
    torch.testing.assert_close(qk[1, 2], 0.25 * q[:, 1, 2] @ k[:, 1, 2].t())
    # rotary embedding preserves norms and is the identity at position 0
    x = torch.randn(2, 4, 6, 16)
    y = _C.fused_apply_rotary_emb(x, x_layout="BHMK", mode="plane")
    torch.testing.assert_close(y.norm(dim=-1), x.norm(dim=-1))
    torch.testing.assert_close(y[:, :, 0], x[:, :, 0])
    yi = _C.fused_apply_rotary_emb(x, x_layout="BHMK", mode="interval")
    torch.testing.assert_close(yi.norm(dim=-1), x.norm(dim=-1))
    pk, pv = torch.randn(2, 4, 3, 8), torch.randn(2, 4, 3, 8)
    k2, v2 = _C.fused_attention_concat_past_key_value(past_key=pk, past_key_layout="BHMK", past_value=pv, past_value_layout="BHMK",
                                                     key=torch.randn(2, 4, 1, 8), key_layout="BHMK", value=torch.randn(2, 4, 1, 8),
                                                     value_layout="BHMK")
    assert k2.shape == (2, 4, 4, 8) and v2.shape == (2, 4, 4, 8)


def test_box_iou_family():
    torch.manual_seed(4)
    x1, y1, x2, y2 = torch.rand(8), torch.rand(8), torch.rand(8), torch.rand(8)
    w1, h1, w2, h2 = torch.rand(8) + 0.1, torch.rand(8) + 0.1, torch.rand(8) + 0.1, torch.rand(8) + 0.1
    b = _C.fused_get_boundding_boxes_coord(x1, y1, w1, h1, x2, y2, w2, h2)
    b1_x1, b1_x2, b1_y1, b1_y2, b2_x1, b2_x2, b2_y1, b2_y2 = b
    inter = _C.fused_get_intersection_area(b1_x1, b1_x2, b2_x1, b2_x2, b1_y1, b1_y2, b2_y1, b2_y2)
    iou = _C.fused_get_iou(w1, h1, w2, h2, inter, 1e-7)
    assert torch.all((iou >= 0) & (iou <= 1 + 1e-5))
    same = _C.fused_get_iou(w1, h1, w1, h1, w1 * h1, 0.0)
    torch.testing.assert_close(same, torch.ones(8))
    c2 = _C.fused_get_convex_diagonal_squared(b1_x1, b1_x2, b2_x1, b2_x2, b1_y1, b1_y2, b2_y1, b2_y2, 1e-8)
    rho2 = _C.fused_get_center_dist(b1_x1, b1_x2, b2_x1, b2_x2, b1_y1, b1_y2, b2_y1, b2_y2)
    torch.testing.assert_close(rho2, (x2 - x1) ** 2 + (y2 - y1) ** 2)
    v = _C.fused_get_ciou_diagonal_angle(w1, h1, w2, h2, 1e-8)
    y, alpha = _C.fused_get_ciou_result(v, iou, rho2, c2, 1e-7)
    torch.testing.assert_close(y, iou - (rho2 / c2 + v * (v / (v - iou + 1 + 1e-7))))
    assert torch.all(c2 >= rho2 - 1e-6)


def test_attention_layouts_roundtrip_and_packing():
    from oneflow_b200.ops import attn_layout as L
    B, H, M, K = 2, 3, 5, 4
    q, k, v = (torch.randn(B, H, M, K) for _ in range(3))
    for layout in ("BHMK", "BMHK", "MBHK", "BM(HK)", "MB(HK)"):
        assert torch.equal(L.unpack(L.pack(q, layout), layout, head_size=K), q), layout
    packed = torch.stack([q, k, v], 3).permute(0, 2, 1, 3, 4).reshape(B, M, H * 3 * K)          # BM(H3K)
    for i, t in enumerate((q, k, v)):
        assert torch.equal(L.unpack(packed, "BM(H3K)", head_size=K, index=i), t)
        assert torch.equal(L.unpack(packed.transpose(0, 1), "MB(H3K)", num_heads=H, index=i), t)
    with pytest.raises(ValueError):
        L.unpack(packed, "BM(H3K)")


def test_concat_past_key_value_layouts():
    B, H, M, K = 2, 3, 4, 8
    pk, pv, nk, nv = (torch.randn(B, H, n, K) for n in (M, M, 1, 1))
    ck, cv = flow._C.fused_attention_concat_past_key_value(
        past_key=pk, past_key_layout="BHMK", past_value=pv.permute(2, 0, 1, 3), past_value_layout="MBHK",
        key=nk.permute(0, 2, 1, 3).reshape(B, 1, H * K), key_layout="BM(HK)", value=nv.permute(0, 2, 1, 3), value_layout="BMHK",
        key_head_size=K)
    assert torch.equal(ck, torch.cat([pk, nk], 2)) and torch.equal(cv, torch.cat([pv, nv], 2).permute(2, 0, 1, 3))
    k0, v0 = flow._C.fused_attention_concat_past_key_value(past_key_layout="BHMK", past_value_layout="BHMK", key=nk, key_layout="BHMK",
                                                          value=nv, value_layout="BHMK")
    assert torch.equal(k0, nk) and torch.equal(v0, nv)


def test_rotary_embedding_modes_and_positions():
    B, H, M, K, rs = 2, 2, 6, 8, 4
    x = torch.randn(B, H, M, K)
    pos = torch.randint(0, 12, (B, 1, M))
    y = flow._C.fused_apply_rotary_emb(x, position_ids=pos, x_layout="BHMK", mode="interval", base=100.0, rotary_size=rs)
    freq = 100.0 ** (-2.0 * torch.arange(rs // 2).float() / rs)
    ang = pos[:, 0, :, None].float() * freq                                           # [B, M, rs/2]
    c, s = ang.cos()[:, None], ang.sin()[:, None]
    e, o = x[..., 0:rs:2], x[..., 1:rs:2]
    assert torch.allclose(y[..., 0:rs:2], e * c - o * s, atol=1e-5) and torch.allclose(y[..., 1:rs:2], o * c + e * s, atol=1e-5)
    assert torch.equal(y[..., rs:], x[..., rs:])                                      # the non-rotary tail passes through
    y2 = flow._C.fused_apply_rotary_emb(x, position_ids=pos, x_layout="BHMK", mode="plane", base=100.0, rotary_size=rs)
    a, b = x[..., :rs // 2], x[..., rs // 2:rs]
    assert torch.allclose(y2[..., :rs // 2], a * c - b * s, atol=1e-5) and torch.allclose(y2[..., rs // 2:rs], b * c + a * s, atol=1e-5)
    # rotations preserve the norm of every pair, whatever the layout the result is asked in
    y3 = flow._C.fused_apply_rotary_emb(x.permute(0, 2, 1, 3).reshape(B, M, H * K), x_layout="BM(HK)", output_layout="MBHK", k_size=K,
                                        mode="interval")
    assert y3.shape == (M, B, H, K) and torch.allclose(y3.norm(dim=-1), x.permute(2, 0, 1, 3).norm(dim=-1), atol=1e-5)


def test_roi_align_matches_torchvision_including_boxes_past_the_border():
    import torchvision
    from oneflow_b200.framework.toplevel_extra import _roi_align_impl
    torch.manual_seed(0)
    x = torch.randn(2, 3, 16, 16)
    rois = torch.tensor([[0, 1., 2., 9., 11.], [1, 0.5, 0.5, 14.2, 8.8], [0, -3., -2., 40., 37.]])
    for aligned in (False, True):
        for sr in (2, -1):
            ref = torchvision.ops.roi_align(x, rois, (5, 5), 0.5, sr, aligned)
            assert torch.allclose(_roi_align_impl(x, rois, (5, 5), 0.5, sr, aligned), ref, atol=1e-5)
            assert torch.allclose(flow.roi_align(x, rois, 0.5, 5, 5, sr, aligned), ref, atol=1e-5)


def test_fused_mlp_chain_matches_separate_layers():
    """flow._C.fused_mlp / nn.FusedMLP (a chain of linear + ReLU layers whose backward folds each ReLU gradient into the next
    data-gradient GEMM on CUDA) give the values and gradients of the plain layer-by-layer statement."""
    import torch
    import oneflow_b200 as flow
    torch.manual_seed(5)
    x = torch.randn(6, 16, requires_grad=True)
    ws = [torch.randn(32, 16, requires_grad=True), torch.randn(24, 32, requires_grad=True), torch.randn(8, 24, requires_grad=True)]
    bs = [torch.randn(32, requires_grad=True), torch.randn(24, requires_grad=True), torch.randn(8, requires_grad=True)]
    for skip in (False, True):
        for t in [x] + ws + bs:
            t.grad = None
        y = flow._C.fused_mlp(x, ws, bs, skip_final_activation=skip)
        y.pow(2).sum().backward()
        got = [t.grad.clone() for t in [x] + ws + bs]
        for t in [x] + ws + bs:
            t.grad = None
        h = x
        for i, (w, b) in enumerate(zip(ws, bs)):
            h = torch.nn.functional.linear(h, w, b)
            if not (skip and i == 2):
                h = torch.relu(h)
        assert torch.allclose(y, h, atol=1e-5)
        h.pow(2).sum().backward()
        for a, t in zip(got, [x] + ws + bs):
            assert torch.allclose(a, t.grad, atol=1e-4)
    m = flow.nn.FusedMLP(16, [32, 24], 8, skip_final_activation=True)
    out = m(x.detach())
    ref = x.detach()
    for i in range(3):
        ref = torch.nn.functional.linear(ref, m.weight(i), m.bias(i))
        if i < 2:
            ref = torch.relu(ref)
    assert torch.allclose(out, ref, atol=1e-5)
