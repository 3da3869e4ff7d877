"""Import paths and the smaller pieces of the public API: dotted ``oneflow.*`` imports, config switches, remat,
sysconfig, mock helpers, extra functionals and modules, schedulers, parameter grouping, persistent table IO (CPU)."""
import importlib

import numpy as np
import pytest
import torch

import oneflow as flow


@pytest.mark.parametrize("path", [
    "oneflow.nn", "oneflow.nn.functional", "oneflow.nn.init", "oneflow.nn.utils", "oneflow.nn.utils.rnn", "oneflow.nn.utils.prune",
    "oneflow.nn.utils.clip_grad", "oneflow.nn.utils.parameters_grouping", "oneflow.nn.utils.skip_init", "oneflow.nn.image",
    "oneflow.nn.qat", "oneflow.nn.graph", "oneflow.nn.parallel", "oneflow.nn.modules.module", "oneflow.nn.modules.utils",
    "oneflow.nn.modules.dataset", "oneflow.nn.optimizer.adam", "oneflow.nn.optimizer.sgd", "oneflow.nn.optimizer.warmup_lr",
    "oneflow.nn.optimizer.cosine_decay_lr", "oneflow.nn.parameter", "oneflow.nn.common_types", "oneflow.optim",
    "oneflow.optim.lr_scheduler", "oneflow.optim.swa_utils", "oneflow.framework.tensor", "oneflow.framework.config_util",
    "oneflow.linalg", "oneflow.fft", "oneflow.special", "oneflow.sysconfig", "oneflow.remat", "oneflow.unittest",
    "oneflow.unittest.env", "oneflow.asyncs", "oneflow.hub", "oneflow.multiprocessing", "oneflow.cuda.amp",
    "oneflow.cuda.type_tensor", "oneflow.backends.cudnn", "oneflow.backends.cuda", "oneflow.utils.data",
    "oneflow.utils.data.distributed", "oneflow.utils.hooks", "oneflow.utils.checkpoint", "oneflow.distributed",
    "oneflow.one_embedding", "oneflow.profiler", "oneflow.mock_torch", "oneflow.autograd", "oneflow.comm", "oneflow.env",
    "oneflow.sbp", "oneflow.amp", "oneflow._oneflow_internal",
])
def test_dotted_import_paths(path):
    assert importlib.import_module(path) is not None


def test_from_imports_give_the_flow_objects():
    from oneflow.framework.tensor import Tensor
    from oneflow.nn.modules.module import Module
    from oneflow.nn.optimizer.adam import Adam
    from oneflow.nn.parameter import Parameter
    from oneflow.nn.utils import clip_grad_norm_
    from oneflow.nn.utils.clip_grad import clip_grad_norm_ as again
    assert Tensor is flow.Tensor and Module is flow.nn.Module and Adam is flow.optim.Adam and again is clip_grad_norm_
    assert isinstance(flow.nn.Parameter(flow.ones(1)), Parameter)
    assert flow.nn.functional.__name__.startswith("oneflow_b200") and flow.nn.init.__name__.startswith("oneflow_b200")
    with pytest.raises(ModuleNotFoundError):
        importlib.import_module("oneflow.no_such_module")


def test_config_switches_and_boxing_namespace():
    from oneflow.framework import config_util as cu
    flow.boxing.nccl.set_fusion_threshold_mbytes(32)
    flow.boxing.nccl.allow_fuse_all_reduce(False)
    flow.boxing.enable_fusion(True)
    flow.backends.cudnn.set_reserved_mem_mbytes(256)
    r = cu.resource()
    assert r["nccl_fusion_threshold_mb"] == 32 and r["nccl_fusion_all_reduce"] is False and r["reserved_device_mem_mbyte"] == 256
    with pytest.raises(TypeError):
        flow.boxing.nccl.set_fusion_threshold_mbytes("big")
    old = flow.backends.cuda.matmul.allow_tf32
    flow.backends.cuda.matmul.allow_tf32 = True
    assert torch.backends.cuda.matmul.allow_tf32 is True
    flow.backends.cuda.matmul.allow_tf32 = old
    with pytest.raises(AssertionError):
        flow.backends.cuda.matmul.nonsense


def test_remat_sysconfig_unittest_env(monkeypatch):
    assert flow.remat.parse_size("2GB") == 2 << 30 and flow.remat.parse_size("1.5 mb") == int(1.5 * 2 ** 20)
    flow.remat.set_budget("512MB")
    assert flow.remat.get_budget() == 512 << 20 and flow.remat.is_enabled()
    assert flow.sysconfig.get_include().endswith("api") and flow.sysconfig.with_cuda() and flow.sysconfig.get_cuda_version() >= 12000
    assert any(f.startswith("-l") for f in flow.sysconfig.get_link_flags())
    monkeypatch.setenv("ONEFLOW_TEST_DEVICE_NUM", "2")
    assert flow.unittest.env.device_num() == 2
    skipped = flow.unittest.skip_unless_1n1d()(type("T", (flow.unittest.TestCase,), {}))
    assert getattr(skipped, "__unittest_skip__", False)
    kept = flow.unittest.skip_unless_1n2d()(type("T", (flow.unittest.TestCase,), {}))
    assert not getattr(kept, "__unittest_skip__", False)


def test_mock_helpers():
    import math
    from oneflow.mock_torch import DummyModule, DynamicMockModule, ModuleWrapper
    d = DummyModule("x")
    assert not d.a.b(1)["k"] and list(d) == []

    class K(d.Base):
        pass
    w = ModuleWrapper(math, lazy=True)
    assert w.pi == math.pi and not w.nothing
    with pytest.raises(AttributeError):
        ModuleWrapper(math).nothing
    m = DynamicMockModule.from_package("json")
    m.hijack("dumps", 5)
    assert m.dumps == 5 and m.loads("1") == 1 and m.decoder is not None


def test_functional_additions():
    import torchvision
    F = flow.nn.functional
    x = torch.randn(5, 7)
    assert torch.allclose(F.quick_gelu(x), x * torch.sigmoid(1.702 * x)) and torch.allclose(F.square_relu(x), x.clamp(min=0) ** 2)
    lab = torch.randint(0, 7, (5,))
    assert torch.allclose(F.sparse_softmax_cross_entropy(lab, x), torch.nn.functional.cross_entropy(x, lab, reduction="none"))
    assert F.interpolate_like(torch.randn(1, 2, 4, 4), torch.randn(1, 2, 8, 6)).shape == (1, 2, 8, 6)
    # the reference's documented example (python/oneflow/framework/docstr/ctc_decode.py)
    lp = torch.tensor([[[-1.54, -1.20, -1.95, -1.65, -1.81], [-1.84, -1.74, -1.58, -1.55, -1.12]],
                       [[-1.68, -1.48, -1.89, -1.30, -2.07], [-1.13, -1.45, -1.24, -1.61, -1.66]],
                       [[-1.56, -1.40, -2.83, -1.67, -1.48], [-1.20, -2.01, -2.05, -1.95, -1.24]],
                       [[-2.09, -1.76, -1.36, -1.67, -1.45], [-1.85, -1.48, -1.34, -2.16, -1.55]]])
    dec, neg = F.ctc_greedy_decoder(lp, torch.tensor([4, 4]))
    assert dec.tolist() == [[1, 3, 1, 2], [0, 2, 0, 0]] and torch.allclose(neg, torch.tensor([[5.26], [4.79]]))
    dec2, neg2 = F.ctc_greedy_decoder(lp, torch.tensor([4, 2]), merge_repeated=False)
    assert dec2.tolist() == [[1, 3, 1, 2], [0, 0, 0, 0]] and abs(neg2[1, 0].item() - 2.25) < 1e-6
    # depend: identity forward, zero gradient to the dependency
    a = torch.randn(3, requires_grad=True)
    b = torch.randn(3, requires_grad=True)
    y = F.depend(a * 2, [b * 3])
    y.sum().backward()
    assert torch.equal(a.grad, torch.full((3,), 2.0)) and torch.equal(b.grad, torch.zeros(3))
    # deformable convolution against torchvision, with groups, offset groups, stride, padding and mask
    torch.manual_seed(0)
    inp, w = torch.randn(2, 8, 9, 11), torch.randn(6, 4, 3, 3)
    off, msk, bias = torch.randn(2, 2 * 2 * 9, 5, 6) * 1.5, torch.rand(2, 2 * 9, 5, 6), torch.randn(6)
    mine = F.deform_conv2d(inp, off, w, bias, stride=(2, 2), padding=(1, 1), mask=msk)
    ref = torchvision.ops.deform_conv2d(inp, off, w, bias, stride=(2, 2), padding=(1, 1), mask=msk)
    assert torch.allclose(mine, ref, atol=1e-4)
    zero = F.deform_conv2d(inp, torch.zeros(2, 18, 9, 11), w[:, :, :, :], None, padding=(1, 1))
    assert torch.allclose(zero, torch.nn.functional.conv2d(inp, w, padding=1, groups=2), atol=1e-4)


def test_small_modules_and_qat_conv():
    x = torch.randn(4, 16)
    assert torch.allclose(flow.nn.QuickGELU()(x), x * torch.sigmoid(1.702 * x))
    assert torch.allclose(flow.nn.SquareReLU()(x), torch.relu(x) ** 2)
    n = flow.nn.RMSLayerNorm(16, eps=1e-6)
    assert torch.allclose(n(x), x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6), atol=1e-6)
    assert torch.equal(flow.nn.AllReduce("cpu:0")(x), x)                      # one rank: the sum is the input
    w = torch.randn(32, 8)
    mapped, sampled, sw = flow.nn.DistributedPariticalFCSample(10)(w, torch.tensor([3, 7, 3]))
    assert sw.shape == (10, 8) and torch.equal(sampled[mapped], torch.tensor([3, 7, 3]))
    torch.manual_seed(0)
    q = flow.nn.QatConv2d(3, 5, 3, padding=1, quantization_bit=8)
    ref = torch.nn.Conv2d(3, 5, 3, padding=1)
    ref.load_state_dict({k: v for k, v in q.state_dict().items() if k in ("weight", "bias")})
    img = torch.randn(2, 3, 8, 8)
    out = q(img)
    assert out.shape == (2, 5, 8, 8) and (out - ref(img)).abs().max() < 0.15 and not torch.equal(out, ref(img))
    out.sum().backward()
    assert q.weight.grad is not None and q.weight.grad.abs().sum() > 0       # straight-through gradient
    assert flow.nn.QatConv1d(2, 2, 3)(torch.randn(1, 2, 9)).shape == (1, 2, 7)
    assert flow.nn.qat.QatConv3d(1, 2, 3)(torch.randn(1, 1, 5, 5, 5)).shape == (1, 2, 3, 3, 3)


def test_warmup_lr_matches_reference_schedule():
    p = [torch.nn.Parameter(torch.zeros(1))]

    def run(prefix):
        o = flow.optim.SGD(p, lr=0.001)
        cd = flow.optim.lr_scheduler.CosineDecayLR(o, decay_steps=5, alpha=0.1)
        w = flow.optim.lr_scheduler.WarmUpLR(cd, warmup_factor=0.5, warmup_iters=2, warmup_method="linear", warmup_prefix=prefix)
        out = []
        for _ in range(7):
            out.append(o.param_groups[0]["lr"])
            o.step()
            w.step()
        return out

    cos = lambda s: 0.001 * (0.9 * 0.5 * (1 + np.cos(np.pi * min(s, 5) / 5)) + 0.1)  # noqa: E731
    a = run(False)   # the decay runs underneath; the warm-up ends on the decay's value at step 2
    assert np.allclose(a, [0.0005, 0.0005 + (cos(2) - 0.0005) / 2, cos(2), cos(3), cos(4), cos(5), cos(6)], atol=1e-9)
    b = run(True)    # the decay starts after the warm-up
    assert np.allclose(b, [0.0005, 0.00075, cos(0), cos(1), cos(2), cos(3), cos(4)], atol=1e-9)
    o = flow.optim.SGD(p, lr=0.001)
    c = flow.optim.lr_scheduler.WarmUpLR(o, warmup_factor=0.5, warmup_iters=5, warmup_method="constant")
    seen = []
    for _ in range(7):
        seen.append(o.param_groups[0]["lr"])
        o.step()
        c.step()
    assert np.allclose(seen, [0.0005] * 5 + [0.001] * 2)
    with pytest.raises(ValueError):
        flow.optim.lr_scheduler.WarmUpLR(o, warmup_iters=0)


def test_contiguous_params_group():
    torch.manual_seed(0)
    m = torch.nn.Sequential(torch.nn.Linear(5, 7), torch.nn.Linear(7, 3))
    ref = [p.detach().clone() for p in m.parameters()]
    g = flow.nn.utils.ContiguousParamsGroup([list(m[0].parameters()), list(m[1].parameters())], group_on_current_buffer=False)
    assert len(g.grouped_parameters) == 2 and all(t.numel() % 128 == 0 for t in g.grouped_parameters)
    assert all(torch.equal(a, b) for a, b in zip(ref, m.parameters()))
    m(torch.randn(4, 5)).sum().backward()
    assert m[0].weight.grad.data_ptr() == g.grouped_parameters_grad[0].data_ptr() and g.grouped_parameters_grad[0].abs().sum() > 0
    torch.optim.SGD(g.grouped_parameters, lr=0.1).step()                     # one flat update moves the views
    assert not torch.equal(m[0].weight, ref[0]) and not torch.equal(m[1].bias, ref[3])
    g2 = flow.nn.utils.ContiguousParamsGroup([[m[0].weight, m[0].bias], [m[1].bias]])   # regroup on the existing buffers
    assert [t.numel() for t in g2.grouped_parameters] == [256, 128]
    assert flow.nn.init.calc_fan((8, 4, 3, 3), "fan_out", "channels_first") == 72.0
    assert flow.nn.init.calc_fan((8, 3, 3, 4), "fan_in", "channels_last") == 36.0
    assert flow.nn.init.get_data_format("NCHW") == "channels_first" and flow.nn.init.get_data_format("NHWC") == "channels_last"


def test_persistent_table_reader_writer(tmp_path):
    paths = [str(tmp_path / "t0"), str(tmp_path / "t1")]
    k = np.arange(1000, dtype=np.int64) * 7
    v = np.random.RandomState(0).rand(1000, 8).astype(np.float32)
    with flow.one_embedding.make_persistent_table_writer(paths, "snap", flow.int64, flow.float32, 8) as w:
        w.write(k[:600], v[:600])
        w.write(k[600:], v[600:])
    got = {}
    with flow.one_embedding.make_persistent_table_reader(paths, "snap", flow.int64, flow.float32, 8) as r:
        for kk, vv in r:
            assert kk.dtype == np.int64 and vv.shape == (kk.size, 8)
            got.update({int(a): b for a, b in zip(kk, vv)})
    assert len(got) == 1000 and all(np.array_equal(got[int(a)], b) for a, b in zip(k, v))
    init = flow.one_embedding.make_trunc_normal_initializer(mean=0, std=0.01, a=-0.02, b=0.02)
    assert init["type"] == "trunc_normal" and init["b"] == 0.02


def test_autograd_and_profiler_names():
    j = flow.autograd.jacobian(lambda t: t ** 2, torch.tensor([1.0, 2.0]))
    assert torch.allclose(j, torch.diag(torch.tensor([2.0, 4.0]))) and flow.autograd.is_grad_enabled()
    flow.profiler.range_push("r")
    flow.profiler.range_pop()
    assert flow.profiler.kineto_available() in (True, False) and flow.profiler.ProfilerAction is not None
    with flow.asyncs.thread(flow.asyncs.Thread()) as t:
        y = flow.ones(2) + 1
    t.join()
    assert y.tolist() == [2.0, 2.0]


def test_tensor_methods_of_the_reference():
    x = flow.randn(4, 6)
    assert x.cast(flow.int32).dtype == torch.int32 and x.is_lazy is False and x.is_consistent is False
    assert torch.allclose(x.silu(), torch.nn.functional.silu(x)) and torch.allclose(x.mish(), torch.nn.functional.mish(x))
    assert torch.allclose(x.softplus(beta=2), torch.nn.functional.softplus(x, 2)) and torch.allclose(x.gelu(), torch.nn.functional.gelu(x))
    w = flow.empty(8, 8).xavier_uniform_()
    assert w.abs().max() <= (6 / 16) ** 0.5 + 1e-6
    assert flow.empty(64).trunc_normal_(std=0.02, a=-0.04, b=0.04).abs().max() <= 0.04
    assert not x.is_offloaded()
    with pytest.warns(UserWarning):
        x.offload()                                           # a host tensor has nowhere to go
    with pytest.raises(RuntimeError):
        x.global_to_global(sbp=flow.sbp.broadcast)
    pl = flow.placement("cpu", [0])
    g = x.local_to_global(pl, flow.sbp.broadcast)
    assert g.is_global and g.is_consistent and g.global_to_global(sbp=flow.sbp.broadcast) is g


def test_graph_sharing_dynamic_shapes_and_description():
    class G(flow.nn.Graph):
        @flow.nn.Graph.with_dynamic_input_shape(size=2)
        def __init__(self):
            super().__init__()
            self.m = torch.nn.Linear(4, 2)

        def build(self, x):
            return self.m(x)

    g = G()
    g.enable_shared()
    assert not g.is_compiled
    assert [g(torch.randn(n, 4)).shape[0] for n in (3, 5, 7)] == [3, 5, 7] and len(g._dynamic_metas) == 2 and g.is_compiled
    assert "Linear" in g._ops_repr()[0] and g._graph_proto["blocks"]["m"]["parameters"] == 10 and g._compiled_graph_proto["compiled"]
    with pytest.raises(RuntimeError):
        g.enable_shared()                                     # only before the first call

    class H(flow.nn.Graph):
        def __init__(self):
            super().__init__()
            self.m = torch.nn.Linear(4, 2)

        def build(self, x):
            return self.m(x)

    h = H()
    h.share_from(g)
    h(torch.randn(3, 4))
    with pytest.raises(RuntimeError):
        h(torch.randn(4, 4))                                  # a plain graph keeps its first input signature
    with pytest.raises(RuntimeError):
        H().share_from(H())                                   # the source was never enabled for sharing
    o = flow.optim.SGD([torch.nn.Parameter(torch.ones(2))], lr=0.1)
    assert o.support_sparse() is False and hasattr(flow.optim.Optimizer, "clip_grad")


def test_generator_per_device_streams():
    """``flow.Generator``: one seed for every device, ``"auto"`` follows the consuming op, and the process-wide
    generator is the one behind ``flow.get_rng_state`` (reference: python/oneflow/test/modules/test_generator.py)."""
    import oneflow
    auto, cpu = flow.Generator(device="auto"), flow.Generator(device="cpu")
    assert auto.initial_seed() == cpu.initial_seed()
    with pytest.raises(RuntimeError):
        flow.Generator(device="invalid")
    flow.Generator(device="cpu:1000")
    g = flow.Generator()
    assert g.manual_seed(7) is g and g.initial_seed() == 7
    a = flow.rand(8, generator=g)
    g.manual_seed(7)
    assert torch.equal(a, flow.rand(8, generator=g))
    assert flow.randperm(6, generator=g).sort().values.tolist() == list(range(6))
    out = flow._C.dropout(flow.ones(1000), p=0.5, training=True, generator=flow.Generator(), addend=None)
    assert 300 < int((out == 0).sum()) < 700
    d = flow.default_generator
    assert d.seed() == d.initial_seed()
    assert torch.equal(d.get_state(), flow.get_rng_state())
    flow.randn(10, generator=d)
    assert torch.equal(d.get_state(), flow.get_rng_state())
    assert issubclass(oneflow._oneflow_internal.exception.RuntimeError, Exception)


def test_nhwc_layers_by_environment(monkeypatch):
    """``ONEFLOW_ENABLE_NHWC=1``: conv / pooling / batch norm take [N, H, W, C], the conv weight is
    [Cout, kH, kW, Cin]; results equal the NCHW layers on permuted data."""
    monkeypatch.setenv("ONEFLOW_ENABLE_NHWC", "1")
    x = torch.randn(2, 12, 12, 3)
    nchw = x.permute(0, 3, 1, 2)
    kw = dict(kernel_size=3, stride=(1, 2), padding=(0, 1), ceil_mode=True)
    assert torch.equal(flow.nn.MaxPool2d(**kw)(x), torch.nn.MaxPool2d(**kw)(nchw).permute(0, 2, 3, 1))
    assert torch.allclose(flow.nn.AvgPool2d(2)(x), torch.nn.AvgPool2d(2)(nchw).permute(0, 2, 3, 1))
    c = flow.nn.Conv2d(3, 8, 3, padding=1)
    assert tuple(c.weight.shape) == (8, 3, 3, 3) and c.channel_pos == "channels_last"
    ref = torch.nn.Conv2d(3, 8, 3, padding=1)
    ref.load_state_dict({"weight": c.weight.detach().permute(0, 3, 1, 2), "bias": c.bias.detach()})
    y = c(x)
    assert torch.allclose(y, ref(nchw).permute(0, 2, 3, 1), atol=1e-5)
    y.sum().backward()
    assert c.weight.grad.shape == c.weight.shape
    rb = torch.nn.BatchNorm2d(3)(nchw).permute(0, 2, 3, 1)
    assert torch.allclose(flow.nn.BatchNorm2d(3)(x), rb, atol=1e-5)
    assert torch.allclose(flow.nn.functional.batch_norm(x, None, None, training=True), rb, atol=1e-5)
    w = flow.nn.init.kaiming_normal_(torch.empty(64, 3, 3, 16), mode="fan_out")
    assert abs(float(w.std()) - (2 / (64 * 9)) ** 0.5) < 0.01
    monkeypatch.setenv("ONEFLOW_ENABLE_NHWC", "0")
    c2 = flow.nn.Conv2d(3, 8, 3, padding=1)
    assert c2.channel_pos == "channels_first" and c2(nchw).shape == (2, 8, 12, 12)
    c2.to_memory_format(flow.channels_last)
    assert c2.channel_pos == "channels_last" and c2(x).shape == (2, 12, 12, 8)


def test_whole_module_save_load_and_module_semantics(tmp_path):
    """A module saved whole comes back runnable; ``state_dict`` hands out the parameters themselves; backward hooks
    see ``TensorTuple`` arguments and may return gradients of another dtype."""
    from oneflow._oneflow_internal import TensorTuple
    m = torch.nn.Sequential(flow.nn.Conv2d(3, 4, 3), torch.nn.ReLU())
    flow.save(m, str(tmp_path / "m"))
    m2 = flow.load(str(tmp_path / "m"))
    x = torch.randn(1, 3, 5, 5)
    assert torch.equal(m(x), m2(x))
    with open(tmp_path / "m", "rb") as f:
        assert torch.equal(flow.load(f)(x), m(x))
    assert m.state_dict()["0.weight"] is m[0].weight
    assert not m.state_dict(keep_vars=False)["0.weight"].requires_grad
    seen = []

    def hook(mod, gin, gout):
        seen.append((isinstance(gin, TensorTuple), isinstance(gout, TensorTuple)))
        return (torch.tensor([1, 1]),)
    r = flow.nn.ReLU()
    r.register_full_backward_hook(hook)
    x0 = torch.tensor([1.0, -1.0], requires_grad=True)
    r(x0 + 1).sum().backward()
    assert seen == [(True, True)] and x0.grad.tolist() == [1.0, 1.0]

    class F(flow.autograd.Function):
        @staticmethod
        def forward(ctx, a):
            ctx.save_for_backward(a.clone())
            F.ctx = ctx
            return a * 2

        @staticmethod
        def backward(ctx, g):
            return g * 2
    out = F.apply(torch.randn(3, requires_grad=True))
    assert F.ctx._is_data_valid()
    out.sum().backward()
    assert not F.ctx._is_data_valid()
    assert flow.device("mock").type == "mock" and flow.placement("mock", [0]).type == "mock"


def test_global_rnn_batch_first_and_type_as():
    P = flow.placement("cpu", [0])
    mt = torch.nn.LSTM(2, 3, batch_first=True)
    mf = flow.nn.LSTM(2, 3, batch_first=True)
    mf.load_state_dict({k: v.detach().numpy() for k, v in mt.state_dict().items()})
    mf = mf.to_global(P, flow.sbp.broadcast)
    x = torch.rand(5, 7, 2)
    xg = x.clone().requires_grad_().to_global(P, flow.sbp.broadcast)
    out, _ = mf(xg)
    ref, _ = mt(x)
    assert out.shape == ref.shape and torch.allclose(out.to_local(), ref, atol=1e-5)
    out.sum().backward()
    t = xg.detach().transpose(0, 1)
    assert not t.to_local().is_contiguous() and t.contiguous().to_local().is_contiguous()
    tgt = flow.ones(2, 2, dtype=flow.int32).to_global(P, flow.sbp.broadcast)
    g = torch.rand(2, 2).type_as(tgt)
    assert g.is_global and g.dtype == flow.int32 and g.placement == tgt.placement
    loc = tgt.type_as(torch.rand(1))
    assert not loc.is_global and loc.dtype == torch.float32
    assert torch.ones(2, dtype=torch.int8).type(flow.Tensor).dtype == torch.float32


def test_mock_torch_import_redirection():
    """Under ``mock_torch.enable()`` an ``import torch`` in user code gives views of this framework's modules named
    ``oneflow...``; ``disable()`` gives the library back, also to module-valued names of the calling scope."""
    import subprocess
    import sys
    code = r'''
import oneflow as flow, oneflow.mock_torch as mock
with mock.enable():
    import torch, torch.nn, torch.version
with mock.disable():
    import torch, torch.nn, torch.version
real = torch
assert torch.__package__ == "torch"
mock.enable()
assert torch.__package__ == "oneflow" and torch.nn.__package__ == "oneflow.nn", (torch.__package__, torch.nn.__package__)
assert torch.version.__version__ == flow.__version__
from torch import nn
assert nn.__package__ == "oneflow.nn" and nn.Linear(2, 2)(torch.ones(1, 2)).shape == (1, 2)
try:
    from torch import noexist
    raise SystemExit("no error")
except ImportError as e:
    assert "cannot import name 'noexist' from 'oneflow'" in str(e), e
try:
    import torch.noexist
    raise SystemExit("no error")
except ModuleNotFoundError as e:
    assert "oneflow.noexist is not implemented" in str(e), e
mock.disable()
assert torch is real and torch.nn.__package__ == "torch.nn"
with mock.enable(lazy=True):
    from torch import not_exist
    assert not_exist.__name__ == "oneflow.not_exist" and not_exist.x.__name__ == "oneflow.not_exist.x"
    assert not torch.not_exist and list(torch.not_exist) == [] and not isinstance(int, torch._six.string_class)
    with mock.disable():
        assert torch.__package__ == "torch"
    assert torch.__package__ == "oneflow"
assert torch.__package__ == "torch" and torch.ones(2).sum().item() == 2.0
print("MOCK OK")
'''
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300)
    assert "MOCK OK" in out.stdout, out.stdout + out.stderr


def test_graph_private_schedule_inputs_and_proto(tmp_path, monkeypatch):
    """nn.Graph advances its own copy of the LR schedule (the caller's scheduler stays put), logs ``step, lr`` in
    debug mode, keeps in-place writes of ``build`` off the caller's inputs and fills ``config.proto``."""
    monkeypatch.chdir(tmp_path)
    monkeypatch.setenv("ONEFLOW_DEBUG_MODE", "1")
    m = torch.nn.Linear(4, 2)
    opt = flow.optim.SGD(m.parameters(), lr=0.1)
    sch = flow.optim.lr_scheduler.StepLR(opt, step_size=2, gamma=0.5)

    class G(flow.nn.Graph):
        def __init__(self):
            super().__init__()
            self.m = m
            self.add_optimizer(opt, lr_sch=sch)

        def build(self, x):
            x += 1.0
            loss = self.m(x).sum()
            loss.backward()
            return x

    g = G()
    x = torch.zeros(3, 4)
    for _ in range(5):
        out = g(x)
    assert torch.equal(x, torch.zeros(3, 4)) and torch.equal(out, torch.ones(3, 4))
    assert sch.last_step == 0 and sch.get_last_lr() == [0.1]
    import glob
    import os
    rows = open(glob.glob(f"log/*/{os.getpid()}-train_step2lr.csv")[0]).read().strip().splitlines()[1:]
    assert [float(r.split(",")[1]) for r in rows] == [0.1, 0.1, 0.05, 0.05, 0.025]
    proto = g.config.proto
    assert proto["optimizer_conf"][0]["type"] == "SGD" and proto["optimizer_conf"][0]["lr_scheduler"] == "StepLR"
    assert g._filter_states() == ["m.weight", "m.bias"] and g._is_compiled
    fx = flow.fx.symbolic_trace(torch.nn.Sequential(flow.nn.Conv2d(3, 4, 3), torch.nn.ReLU()))
    assert [n.op for n in fx.graph.nodes] == ["placeholder", "call_module", "call_module", "output"]
