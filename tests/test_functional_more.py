"""flow._C: the long tail of functional ops, each against a plain statement of its definition
(reference signatures: oneflow/core/functional/functional_api.yaml)."""
import math

import numpy as np
import pytest
import torch

import oneflow as flow

C = flow._C


def test_every_forward_functor_of_the_reference_resolves():
    names = """abs add addmm arange argmax batch_matmul bias_add broadcast_like cast clamp concat conv2d ctc_loss dropout
    embedding expand flatten gather gelu layer_norm matmul max_pool2d normalization pad reduce_sum reshape slice softmax
    sparse_softmax_cross_entropy split stack transpose tril where one_embedding_id_shuffle fused_dot_feature_interaction
    fused_multi_head_attention_inference multi_tensor_adam_update upsample_bilinear_2d fft_c2c deform_conv2d""".split()
    assert [n for n in names if not hasattr(C, n)] == []


def test_inplace_and_elementwise():
    a = torch.tensor([1.0, 4.0, -2.0])
    assert C.mul_(a.clone(), 2).tolist() == [2.0, 8.0, -4.0]
    assert C.addcmul_(a.clone(), a, a, value=0.5).tolist() == [1.5, 12.0, 0.0]
    assert C.addcdiv_(a.clone(), a, torch.tensor([2.0, 2.0, 2.0]), value=2).tolist() == [2.0, 8.0, -4.0]
    assert C.greater_(a.clone(), 0).tolist() == [1.0, 1.0, 0.0]
    assert C.trunc_divide(torch.tensor([7.0, -7.0]), 2).tolist() == [3.0, -3.0]
    assert C.reciprocal_no_nan(torch.tensor([2.0, 0.0])).tolist() == [0.5, 0.0]
    assert C.not_equal_zero(torch.tensor([0.0, 3.0])).tolist() == [0.0, 1.0]
    assert C.rint(torch.tensor([0.5, 1.5, 2.4])).tolist() == [0.0, 2.0, 2.0]
    assert torch.allclose(C.trigamma(torch.tensor([1.0])), torch.tensor([math.pi ** 2 / 6]))
    assert torch.allclose(C.zeta(torch.tensor([2.0]), torch.tensor([1.0])), torch.tensor([math.pi ** 2 / 6]))
    x = torch.randn(3, 4)
    assert torch.allclose(C.sqrt_square_sum(x), x.norm()) and torch.allclose(C.l2_normalize(x, 1).norm(dim=1), torch.ones(3))
    assert C.T(torch.zeros(2, 3, 4)).shape == (4, 3, 2)
    assert torch.allclose(C.fast_gelu(x), torch.nn.functional.gelu(x, approximate="tanh"))
    assert torch.allclose(C.bias_add(torch.zeros(2, 3, 4), torch.arange(3.0), axis=1)[0, :, 0], torch.arange(3.0))


def test_reductions_and_like_ops():
    x = torch.arange(24.0).reshape(2, 3, 4)
    assert torch.equal(C.reduce_sum(x, [0, 2]), x.sum((0, 2))) and C.reduce_sum(x).item() == 276.0
    assert torch.equal(C.reduce_mean(x, [1], True), x.mean(1, keepdim=True))
    assert torch.equal(C.reduce_prod(x + 1, [0, 1]), (x + 1).prod(0).prod(0))
    assert torch.equal(C.reduce_max(x, [1, 2]), x.amax((1, 2))) and torch.equal(C.reduce_min(x, [0]), x.amin(0))
    assert C.reduce_any(x > 22).item() and not C.reduce_all(x > 0).item()
    assert C.reduce_nansum(torch.tensor([1.0, float("nan")])).item() == 1.0
    out, mask, count = C.reduce_max_device_stage(torch.tensor([[1.0, 3.0, 3.0]]), [1])
    assert out.tolist() == [[3.0]] and mask.tolist() == [[0, 1, 1]] and count.tolist() == [[2]]
    g, m = C.reduce_max_global_stage(torch.tensor([[3.0, 5.0]]), torch.tensor([[2, 1]]), [1])
    assert g.tolist() == [5.0] and m.tolist() == [[0, 1]]
    big = torch.ones(4, 3, 5)
    assert C.broadcast_reduce_sum_like(big, torch.zeros(3, 1)).tolist() == [[20.0]] * 3
    assert C.reduce_sum_like(big, torch.zeros(3), [0, 2]).tolist() == [20.0] * 3
    assert C.reshape_like(torch.arange(6), torch.zeros(2, 3)).shape == (2, 3) and C.cast_like(x, torch.zeros(1, dtype=torch.int32)).dtype == torch.int32
    parts = C.split_like(torch.arange(5), [torch.zeros(2), torch.zeros(3)], 0)
    assert [p.tolist() for p in parts] == [[0, 1], [2, 3, 4]]


def test_shape_helpers():
    x = torch.zeros(3, 4)
    assert C.expand_dims(x, 1).shape == (3, 1, 4) and C.unsqueeze_multiple(x, [1, 3], 4).shape == (1, 3, 1, 4)
    assert C.squeeze_(torch.zeros(1, 3, 1), [0, 2]).shape == (3,)
    t = torch.arange(12).reshape(3, 4).t()
    assert C.contiguous_(t).is_contiguous()
    assert C.repeat_interleave_index(torch.tensor([2, 1, 3]), torch.tensor([2, 3, 6]), 0).tolist() == [0, 0, 1, 2, 2, 2]
    assert C.arg_sort(torch.tensor([[3.0, 1.0, 2.0]]), "DESCENDING").tolist() == [[0, 2, 1]]
    assert C.eye_(torch.ones(2, 3)).tolist() == [[1, 0, 0], [0, 1, 0]]
    assert C.constant([2, 2], 3, dtype=torch.int32).tolist() == [[3, 3], [3, 3]]
    assert C.tensor_constant([2], torch.tensor(1.5), dtype=torch.float32).tolist() == [1.5, 1.5]
    with pytest.raises(RuntimeError):
        C.throw_error(x)


def test_scatter_gather_segment():
    idx = torch.tensor([[0, 1], [2, 0], [0, 1]])
    out = C.scatternd(idx, torch.tensor([1.0, 2.0, 3.0]), [3, 2])
    assert out.tolist() == [[0, 4.0], [0, 0], [2.0, 0]]
    assert C.scatterndlike(torch.zeros(3, 2), torch.tensor([1.0, 2.0, 3.0]), idx).tolist() == out.tolist()
    upd = C.tensor_scatter_nd_update(torch.ones(3, 2), idx[:2], torch.tensor([5.0, 6.0]))
    assert upd.tolist() == [[1, 5.0], [1, 1], [6.0, 1]]
    base = torch.ones(2, 3)
    assert C.scatter_mul(base, 1, torch.tensor([[0], [2]]), torch.tensor([[3.0], [4.0]])).tolist() == [[3, 1, 1], [1, 1, 4]]
    assert C.scatter_update(base, 1, torch.tensor([[0], [2]]), 7.0).tolist() == [[7, 1, 1], [1, 1, 7]]
    assert C.dim_gather(torch.tensor([[1, 2], [3, 4]]), 1, torch.tensor([[1], [0]])).tolist() == [[2], [3]]
    data = torch.tensor([[1.0, 2.0], [3.0, 4.0], [5.0, 6.0]])
    assert C.unsorted_segment_sum(data, torch.tensor([1, 0, 1]), 0, 2).tolist() == [[3, 4], [6, 8]]
    assert C.unsorted_batch_segment_sum(torch.tensor([[1.0, 2.0, 3.0]]), torch.tensor([[1, 1, 0]]), 2).tolist() == [[3.0, 3.0]]


def test_linalg_fft_pads_resampling():
    a, b = torch.randn(2, 3, 4), torch.randn(2, 5, 4)
    assert torch.allclose(C.batch_matmul(a, b, transpose_b=True, alpha=2.0), 2 * a @ b.transpose(1, 2))
    m, v = torch.randn(3, 4), torch.randn(4)
    u = torch.randn(3)
    assert torch.allclose(C.matrix_vector_product(m, v), m @ v) and torch.allclose(C.vector_matrix_product(u, m), u @ m, atol=1e-6)
    assert torch.allclose(C.vector_norm(m, 2, [1]), m.norm(dim=1)) and torch.allclose(C.matrix_norm(m, "fro", [0, 1]), m.norm())
    sq = torch.randn(3, 3) + 3 * torch.eye(3)
    assert torch.allclose(C.inv(sq) @ sq, torch.eye(3), atol=1e-4)
    x = torch.randn(4, 8)
    assert torch.allclose(C.fft_c2c(x.to(torch.complex64), dims=[1]), torch.fft.fft(x, dim=1), atol=1e-5)
    assert torch.allclose(C.fft_r2c(x, dims=[1], onesided=True), torch.fft.rfft(x, dim=1), atol=1e-5)
    assert torch.allclose(C.irfft(C.rfft(x), n=8), x, atol=1e-5) and torch.allclose(C.ifft2(C.fft2(x)).real, x, atol=1e-5)
    assert torch.allclose(C.fft_c2r(torch.fft.rfft(x, dim=1), n=[8], dims=[1], forward=False), x, atol=1e-5)
    img = torch.randn(1, 2, 4, 5)
    assert C.constant_pad(img, [1, 1, 2, 0], 9.0).shape == (1, 2, 6, 7) and C.reflection_pad(img, [1, 1, 1, 1]).shape == (1, 2, 6, 7)
    assert C.upsample_nearest_2d(img, 2.0, 2.0).shape == (1, 2, 8, 10)
    assert torch.allclose(C.upsample_bilinear_2d(img, 0.0, 0.0, True, [8, 10]),
                          torch.nn.functional.interpolate(img, size=(8, 10), mode="bilinear", align_corners=True))
    assert C.upsample_linear_1d(torch.randn(1, 2, 4), 2.0).shape == (1, 2, 8)
    assert C.upsample_trilinear_3d(torch.randn(1, 1, 2, 2, 2), 2.0, 2.0, 2.0).shape == (1, 1, 4, 4, 4)
    w = torch.randn(2, 3, 3, 3)
    assert torch.allclose(C.deconv2d(img, w, None, 2, 1), torch.nn.functional.conv_transpose2d(img, w, None, 2, 1))
    pooled = C.avg_pool2d_nhwc(torch.ones(1, 1, 3, 3), [2, 2], [2, 2], "same", [0, 0], [1, 1])
    assert pooled.tolist() == [[[[1.0, 1.0], [1.0, 1.0]]]]                        # padded cells do not dilute the mean


def test_norms_losses_quantization():
    x = torch.randn(6, 4, 3, 3)
    mean, var = torch.zeros(4), torch.ones(4)
    y = C.normalization(x, mean, var, torch.ones(4), torch.zeros(4), 1, 1e-5, 0.9, True)
    assert torch.allclose(y.mean((0, 2, 3)), torch.zeros(4), atol=1e-5)
    assert torch.allclose(mean, 0.1 * x.mean((0, 2, 3)), atol=1e-5)                 # momentum weights the old value
    z = C.normalization_add_relu(x, torch.ones_like(x), None, None, torch.ones(4), torch.zeros(4), 1, 1e-5, 0.9, True)
    assert torch.allclose(z, torch.relu(y + 1), atol=1e-5)
    ln = C.layer_norm_affine(x, torch.full((3, 3), 2.0), torch.zeros(3, 3), 2, 2, 1e-5)
    assert torch.allclose(ln, 2 * torch.nn.functional.layer_norm(x, (3, 3)), atol=1e-5)
    p = torch.softmax(torch.randn(5, 7), -1)
    lab = torch.randint(0, 7, (5,))
    assert torch.allclose(C.sparse_cross_entropy(p, lab, 7), -torch.log(p[torch.arange(5), lab]))
    logits = torch.randn(5, 7)
    assert torch.allclose(C.softmax_cross_entropy(logits, p), -(p * torch.log_softmax(logits, -1)).sum(-1), atol=1e-6)
    assert torch.allclose(C.binary_cross_entropy_with_logits_loss(logits, (p > 0.1).float(), None, None, "mean"),
                          torch.nn.functional.binary_cross_entropy_with_logits(logits, (p > 0.1).float()))
    scale, zp = C.min_max_observer(logits, "google", 8, "symmetric", True)
    fq = C.fake_quantization(logits, scale, zp, "google", 8, "symmetric")
    assert (fq - logits).abs().max() <= scale.item() / 2 + 1e-6
    # group-wise dequantisation: int8 symmetric and packed uint4 with zero points
    q = torch.randint(-127, 127, (4, 8), dtype=torch.int8)
    s = torch.rand(4, 2) + 0.5
    assert torch.allclose(C.groupwise_dequantize(q, s, group_dim=1), q.float() * s.repeat_interleave(4, 1))
    nib = torch.randint(0, 16, (4, 8))
    packed = ((nib[:, 0::2] << 4) | nib[:, 1::2]).to(torch.uint8)
    zero = torch.randint(0, 16, (4, 2)).float()
    deq = C.groupwise_dequantize(packed, s, zero=zero, num_bits=4, symmetric=False, group_dim=1)
    assert torch.allclose(deq, (nib.float() - zero.repeat_interleave(4, 1)) * s.repeat_interleave(4, 1))
    xin = torch.randn(3, 8)
    assert torch.allclose(C.fused_linear_with_groupwise_quantized_weight(xin, q, s, group_dim=1),
                          xin @ (q.float() * s.repeat_interleave(4, 1)).t(), atol=1e-5)


def test_rnn_cells_and_multi_tensor_updates():
    torch.manual_seed(0)
    cell = torch.nn.LSTMCell(5, 6)
    x, h, c = torch.randn(3, 5), torch.randn(3, 6), torch.randn(3, 6)
    hy, cy, _ = C._fused_lstm_cell(x @ cell.weight_ih.t(), h @ cell.weight_hh.t(), c, cell.bias_ih, cell.bias_hh)
    rh, rc = cell(x, (h, c))
    assert torch.allclose(hy, rh, atol=1e-6) and torch.allclose(cy, rc, atol=1e-6)
    gru = torch.nn.GRUCell(5, 6)
    gy, _ = C._fused_gru_cell(x @ gru.weight_ih.t(), h @ gru.weight_hh.t(), h, gru.bias_ih, gru.bias_hh)
    assert torch.allclose(gy, gru(x, h), atol=1e-6)
    ws = [torch.randn(4), torch.randn(2, 3)]
    gs = [torch.randn(4), torch.randn(2, 3)]
    ref = [w - 0.1 * (g * 0.5 + 0.0) - 0.1 * 0.01 * w for w, g in zip(ws, gs)]
    C.multi_tensor_sgd_update(ws, gs, 0.5, 0.01, 0.1)
    assert all(torch.allclose(a, b, atol=1e-6) for a, b in zip(ws, ref))
    w, g = [torch.randn(5)], [torch.randn(5)]
    m, v = [torch.zeros(5)], [torch.zeros(5)]
    p = torch.nn.Parameter(w[0].clone())
    p.grad = g[0].clone()
    opt = torch.optim.Adam([p], lr=0.01, betas=(0.9, 0.999), eps=1e-8)
    opt.step()
    C.multi_tensor_adam_update(w, g, m, v, 0.01, 0.0, 0.9, 0.999, 1 - 0.9, 1 - 0.999, True, 1.0, 0.0, 1e-8)
    assert torch.allclose(w[0], p.detach(), atol=1e-6)
    ema, model = [torch.zeros(3)], [torch.ones(3)]
    C.multi_tensor_yolov5_weight_update(ema, model, 0.9)
    assert torch.allclose(ema[0], torch.full((3,), 0.1))
    data, sizes = C.pack_padded_sequence(torch.arange(6.0).reshape(2, 3, 1), torch.tensor([3, 1]), True)
    assert sizes.tolist() == [2, 1, 1] and data.reshape(-1).tolist() == [0.0, 3.0, 1.0, 2.0]


def test_one_embedding_stage_ops_single_process():
    opts = flow.one_embedding.make_table_options(flow.one_embedding.make_uniform_initializer(-0.1, 0.1))
    store = flow.one_embedding.make_device_mem_store_options(persistent_path="/tmp/ofb_stage_ops", capacity=4096, size_factor=2)
    emb = flow.one_embedding.MultiTableEmbedding("stage_ops_emb", embedding_dim=4, dtype=flow.float32, key_type=flow.int64,
                                                 tables=[opts, opts], store_options=store)
    ids = torch.tensor([[5, 9], [5, 7], [11, 9]])
    tids = torch.tensor([[0, 1], [0, 1], [0, 1]])
    mat, inv_part, n_cur, cur_ids, cur_tids, cur_inv = C.one_embedding_id_shuffle(ids, tids, 2, "stage_ops_emb")
    assert n_cur.item() == 4 and mat.tolist() == [4]
    lines = C.one_embedding_lookup(n_cur, cur_ids, cur_tids, flow.float32, flow.float32, 8, 4, "stage_ops_emb", "", "", 0)
    assert lines.shape == (4, 8) and lines[:, :4].abs().max() <= 0.1 and lines[:, 4:].abs().sum() == 0
    out = C.one_embedding_embedding_shuffle(lines[:, :4], mat, cur_inv, inv_part, "stage_ops_emb")
    assert out.shape == (6, 4) and torch.equal(out[0], out[2]) and torch.equal(out[1], out[5])       # same key, same row
    assert torch.allclose(out, emb(ids, tids).reshape(6, 4))                                         # == the fused forward
    grad = torch.ones(6, 4)
    ug = C.one_embedding_embedding_gradient_shuffle(grad, mat, cur_inv, inv_part, "stage_ops_emb")
    assert ug.shape == (4, 4) and sorted(ug[:, 0].tolist()) == [1.0, 1.0, 2.0, 2.0]                  # duplicates are summed
    new = C.one_embedding_sgd_update(n_cur, lines, ug, None, None, None, 0.5, 1.0, 0.0, 0.9, 8, 4, "stage_ops_emb")
    assert torch.allclose(new[:, 4:], ug) and torch.allclose(new[:, :4], lines[:, :4] - 0.5 * ug)    # momentum line layout
    C.one_embedding_embedding_put(n_cur, cur_ids, new, "stage_ops_emb", 8)
    again = C.one_embedding_lookup(n_cur, cur_ids, cur_tids, flow.float32, flow.float32, 8, 4, "stage_ops_emb", "", "", 0)
    assert torch.allclose(again, new)
    ada = C.one_embedding_adagrad_update(n_cur, lines, ug, None, None, None, None, 0, 0.1, 1.0, 0.0, 0.0, 1e-10, 8, 4, "x")
    assert torch.allclose(ada[:, 4:], ug * ug) and torch.allclose(ada[:, :4], lines[:, :4] - 0.1 * ug / (ug.abs() + 1e-10), atol=1e-6)
    n, uk, uv, inverse = C.one_embedding_unique_key_value_pair(torch.tensor([3, 3, 4]), torch.tensor([0, 0, 1]), 2, "x")
    assert n.item() == 2 and uk.tolist() == [3, 4] and uv.tolist() == [0, 1] and inverse.tolist() == [0, 0, 1]
