"""ResNet-50 (v1.5: stride on the 3x3 of each down-sampling bottleneck) for NHWC bf16 images, as an explicit
forward / backward engine over a flat parameter store.

Every convolution runs on the tensor cores: 1x1 filters are plain tcgen05 GEMMs on the [N H W, C] view, 3x3 filters
the implicit-GEMM kernels of ops/conv.py, the 7x7 RGB stem an im2col + GEMM; stride 2 is expressed as
(stride-1 conv, subsample) or (subsample, 1x1 conv) so that forward and both gradients stay exact adjoints. Batch
norm uses batch statistics with the residual add and the ReLU fused into its apply kernels. Weight gradients
accumulate in fp32 directly from the GEMM epilogues; the data-parallel all-reduce of a stage's gradients is issued
on a side stream as soon as that stage's backward has finished, and one fused SGD-momentum kernel updates the fp32
master weights and the bf16 model copy.

Reference: the flowvision ResNet-50 that the reference's CI speed test trains (ci/test/test_speed_multi_client.sh:28-43),
python/oneflow/nn/modules/{conv,batchnorm,pooling}.py.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import cnn as N
from ..ops import conv as C
from ..ops import gemm as G
from ..ops import kernels as K
from .gpt import ParamStore


@dataclass
class ResNetConfig:
    layers: Tuple[int, ...] = (3, 4, 6, 3)
    widths: Tuple[int, ...] = (64, 128, 256, 512)
    stem: int = 64
    expansion: int = 4
    num_classes: int = 1000
    image_size: int = 224
    bn_eps: float = 1e-5
    bn_momentum: float = 0.1

    def flops_per_image(self):
        """Forward multiply-adds x 2 x 3 (forward + two gradients), convolutions and the classifier only."""
        s = self.image_size // 2
        total = s * s * 7 * 7 * 3 * self.stem
        s //= 2
        cin = self.stem
        for i, (n, w) in enumerate(zip(self.layers, self.widths)):
            for b in range(n):
                stride = 2 if (b == 0 and i > 0) else 1
                so = s // stride
                total += s * s * cin * w + so * so * 9 * w * w + so * so * w * w * self.expansion
                if b == 0:
                    total += so * so * cin * w * self.expansion
                cin, s = w * self.expansion, so
        total += cin * self.num_classes
        return 6 * total


RESNET50 = ResNetConfig()


def tiny_config(**kw):
    base = dict(layers=(1, 1), widths=(64, 64), stem=64, expansion=2, num_classes=16, image_size=32)
    base.update(kw)
    return ResNetConfig(**base)


class _Conv:
    """Convolution with weights [Cout, R, S, Cin] in the store; stride 1 or 2, padding (R - 1) / 2."""

    def __init__(self, net, name, cin, cout, k, stride=1):
        self.net, self.name, self.cin, self.cout, self.k, self.stride = net, name, cin, cout, k, stride
        net.specs.append((name, (cout, k, k, cin), True, math.sqrt(2.0 / (k * k * cout))))

    def fwd(self, x):
        w = self.net.store.p[self.name]
        self.in_shape = tuple(x.shape)
        if self.stride == 2 and self.k == 1:
            x = N.subsample2(x)
        self.x = x
        y = C.conv_fprop(x, w)
        if self.stride == 2 and self.k > 1:
            self.full_shape = tuple(y.shape)
            y = N.subsample2(y)
        return y

    def bwd(self, dy, need_dx=True, residual=None):
        """``residual`` (shape of the input gradient) is added to the returned gradient."""
        st = self.net.store
        w = st.p[self.name]
        if self.stride == 2 and self.k > 1:
            dy = N.upsample2_zero(dy, self.full_shape)
        C.conv_wgrad(self.x, dy, (self.k, self.k), out=st.g[self.name], accumulate=st.acc_flag(self.name))
        dx = None
        if need_dx:
            fuse = residual is not None and not (self.stride == 2 and self.k == 1)
            dx = C.conv_dgrad(dy, w, residual if fuse else None)
            if self.stride == 2 and self.k == 1:
                dx = N.upsample2_zero(dx, self.in_shape)
            if residual is not None and not fuse:
                dx = K.bias_mask_scale(dx, None, None, 1.0, addend=residual)
        self.x = None
        return dx


class _BN:
    def __init__(self, net, name, c, zero_init=False):
        self.net, self.name, self.c = net, name, c
        net.specs.append((name + ".weight", (c,), False, ("const", 0.0 if zero_init else 1.0)))
        net.specs.append((name + ".bias", (c,), False, ("const", 0.0)))
        net.bn_names.append(name)

    def fwd(self, x, residual=None, relu=True):
        net = self.net
        gamma, beta = net.master(self.name + ".weight"), net.master(self.name + ".bias")
        rm, rv = net.running[self.name]
        self.relu, self.has_res = relu, residual is not None
        if not net.training:
            return N.bn_eval_fwd(x, gamma, beta, rm, rv, residual, relu, net.cfg.bn_eps)
        y, self.mean, self.rstd = N.bn_train_fwd(x, gamma, beta, residual, relu, net.cfg.bn_eps, net.cfg.bn_momentum, rm, rv)
        self.x, self.y = x, (y if relu else None)
        return y

    def bwd(self, dy):
        net = self.net
        gamma = net.master(self.name + ".weight")
        dx, dres, dgamma, dbeta = N.bn_train_bwd(dy, self.x, self.y, self.mean, self.rstd, gamma, self.relu, self.has_res)
        for nm, g in ((self.name + ".weight", dgamma), (self.name + ".bias", dbeta)):
            if net.store.acc_flag(nm):
                net.store.g[nm].add_(g)
            else:
                net.store.g[nm].copy_(g)
        self.x = self.y = None
        return dx, dres


class _Bottleneck:
    def __init__(self, net, name, cin, width, stride, expansion):
        cout = width * expansion
        self.conv1 = _Conv(net, name + ".conv1", cin, width, 1)
        self.bn1 = _BN(net, name + ".bn1", width)
        self.conv2 = _Conv(net, name + ".conv2", width, width, 3, stride)
        self.bn2 = _BN(net, name + ".bn2", width)
        self.conv3 = _Conv(net, name + ".conv3", width, cout, 1)
        self.bn3 = _BN(net, name + ".bn3", cout, zero_init=True)
        self.down = None
        if stride != 1 or cin != cout:
            self.down = (_Conv(net, name + ".downsample.0", cin, cout, 1, stride), _BN(net, name + ".downsample.1", cout))

    def fwd(self, x):
        idn = x
        if self.down is not None:
            idn = self.down[1].fwd(self.down[0].fwd(x), relu=False)
        y = self.bn1.fwd(self.conv1.fwd(x))
        y = self.bn2.fwd(self.conv2.fwd(y))
        return self.bn3.fwd(self.conv3.fwd(y), residual=idn, relu=True)

    def bwd(self, dy):
        d3, dres = self.bn3.bwd(dy)
        d = self.conv3.bwd(d3)
        d, _ = self.bn2.bwd(d)
        d = self.conv2.bwd(d)
        d, _ = self.bn1.bwd(d)
        if self.down is not None:
            dd, _ = self.down[1].bwd(dres)
            dres = self.down[0].bwd(dd)
        return self.conv1.bwd(d, residual=dres)     # identity-branch gradient added in the dgrad GEMM epilogue


class ResNet:
    """Parameters, running statistics and the forward / backward passes of one model replica."""

    def __init__(self, cfg: ResNetConfig, device, seed: int = 0):
        self.cfg, self.device = cfg, torch.device(device)
        self.specs: List[tuple] = []
        self.bn_names: List[str] = []
        self.training = True
        self.stem_cols = (7 * 7 * 3 + 7) // 8 * 8
        self.specs.append(("conv1.weight", (cfg.stem, self.stem_cols), True, math.sqrt(2.0 / (49 * cfg.stem))))
        self.bn1 = _BN(self, "bn1", cfg.stem)
        self.stages: List[List[_Bottleneck]] = []
        cin = cfg.stem
        for i, (n, w) in enumerate(zip(cfg.layers, cfg.widths)):
            blocks = []
            for b in range(n):
                blocks.append(_Bottleneck(self, f"layer{i + 1}.{b}", cin, w, 2 if (b == 0 and i > 0) else 1, cfg.expansion))
                cin = w * cfg.expansion
            self.stages.append(blocks)
        self.feat = cin
        self.classes_pad = (cfg.num_classes + 7) // 8 * 8
        self.specs.append(("fc.weight", (self.classes_pad, cin), True, 0.01))
        self.specs.append(("fc.bias", (self.classes_pad,), False, ("const", 0.0)))
        self.store = ParamStore(self.specs, self.device)
        self.store.init_(seed)
        self.store.p["conv1.weight"][:, 147:].zero_()
        if self.classes_pad != cfg.num_classes:
            self.store.p["fc.weight"][cfg.num_classes:].zero_()
        self.running = {n: (torch.zeros(self._bn_c(n), device=self.device), torch.ones(self._bn_c(n), device=self.device))
                        for n in self.bn_names}
        self._master = None   # fp32 master weights (set by the optimizer); batch norm reads its affine parameters there

    def _bn_c(self, name):
        return self.store.offsets[name + ".weight"][1]

    def bind_master(self, master_flat):
        self._master = master_flat

    def master(self, name):
        o, n, shape = self.store.offsets[name]
        if self._master is None:
            return self.store.p[name].float()
        return self._master[o:o + n].view(shape)

    def stage_param_ranges(self):
        """Element ranges of the flat gradient buffer per backward stage (classifier + layer4 first ... stem last)."""
        groups = [["fc."] + [f"layer{len(self.stages)}."]] + [[f"layer{i}."] for i in range(len(self.stages) - 1, 0, -1)]
        groups[-1] += ["conv1.", "bn1."]
        out = []
        for prefixes in groups:
            spans = sorted((o, o + n) for name, (o, n, _) in self.store.offsets.items() if any(name.startswith(p) for p in prefixes))
            merged = []
            for a, b in spans:
                b = (b + 63) // 64 * 64
                if merged and a <= merged[-1][1]:
                    merged[-1][1] = max(merged[-1][1], b)
                else:
                    merged.append([a, b])
            out.append([(a, min(b, self.store.total)) for a, b in merged])
        return out

    # ------------------------------------------------------------------ passes
    def forward(self, images):
        """images: [N, H, W, 3] bf16 (channels last). Returns logits [N, classes_pad] bf16."""
        cfg = self.cfg
        n = images.shape[0]
        cols, (oh, ow) = N.im2col_small(images, 7, 7, 2, 3, self.stem_cols)
        self.stem_cols_saved = cols if self.training else None
        y = G.gemm(cols, self.store.p["conv1.weight"]).view(n, oh, ow, cfg.stem)
        y = self.bn1.fwd(y)
        self.pool_in_shape = tuple(y.shape)
        y, self.pool_idx = N.maxpool3x3s2_fwd(y)
        for blocks in self.stages:
            for b in blocks:
                y = b.fwd(y)
        self.feat_shape = tuple(y.shape)
        f = N.avgpool_fwd(y)
        self.fc_in = f
        return G.gemm(f, self.store.p["fc.weight"], bias=self.store.p["fc.bias"])

    def backward(self, dlogits, stage_done=None):
        """Gradients of all parameters into store.grad. ``stage_done(i)`` is called after backward stage i
        (0 = classifier + last stage ... ) has produced all its parameter gradients."""
        st = self.store
        G.gemm(dlogits, self.fc_in, a_layout="km", b_layout="kn", out=st.g["fc.weight"], out_dtype=torch.float32,
               accumulate=st.acc_flag("fc.weight"))
        if not st.acc_flag("fc.bias"):
            st.g["fc.bias"].zero_()
        K.column_sum(dlogits, out=st.g["fc.bias"])
        d = G.gemm(dlogits, st.p["fc.weight"], b_layout="kn")
        d = N.avgpool_bwd(d, self.feat_shape)
        for i, blocks in enumerate(reversed(self.stages)):
            for b in reversed(blocks):
                d = b.bwd(d)
            if stage_done is not None and i < len(self.stages) - 1:
                stage_done(i)
        d = N.maxpool3x3s2_bwd(d, self.pool_idx, self.pool_in_shape)
        d, _ = self.bn1.bwd(d)
        G.gemm(d.view(-1, self.cfg.stem), self.stem_cols_saved, a_layout="km", b_layout="kn", out=st.g["conv1.weight"],
               out_dtype=torch.float32, accumulate=st.acc_flag("conv1.weight"))
        self.stem_cols_saved = None
        if stage_done is not None:
            stage_done(len(self.stages) - 1)


class ResNetTrainer:
    """Data-parallel ResNet training: forward, softmax cross-entropy, backward with the per-stage gradient all-reduce
    overlapped on a side stream, fused SGD with momentum."""

    def __init__(self, cfg: ResNetConfig, device, group=None, lr=0.1, momentum=0.9, weight_decay=1e-4, seed: int = 0, overlap=True):
        from ..parallel.engine import FlatSGD
        self.cfg, self.device = cfg, torch.device(device)
        self.net = ResNet(cfg, device, seed)
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.reducer = None
        if self.world > 1:
            from ..parallel.zero import GradAllReduce
            ranks = dist.get_process_group_ranks(group) if group is not None else list(range(self.world))
            self.reducer = GradAllReduce(group, ranks, self.device, io_bytes=64 << 20)
        self.opt = FlatSGD(self.net.store, lr=lr, momentum=momentum, weight_decay=weight_decay)
        self.net.bind_master(self.opt.master)
        self.ranges = self.net.stage_param_ranges()
        self.overlap = overlap and self.device.type == "cuda" and self.reducer is not None
        self.comm_stream = torch.cuda.Stream(device=self.device) if self.overlap else None

    def _reduce_stage(self, i):
        if self.reducer is None:
            return
        grad = self.net.store.grad
        if self.overlap:
            ev = torch.cuda.Event()
            ev.record()
            with torch.cuda.stream(self.comm_stream):
                self.comm_stream.wait_event(ev)
                for a, b in self.ranges[i]:
                    self.reducer.all_reduce_(grad[a:b])
        else:
            for a, b in self.ranges[i]:
                self.reducer.all_reduce_(grad[a:b])

    def train_step(self, images, labels):
        """images [N, H, W, 3] bf16, labels int64 [N]. Returns the mean loss of this rank's batch (device tensor)."""
        net = self.net
        net.training = True
        net.store.start_accumulation()
        n = images.shape[0]
        logits = net.forward(images)
        real = logits if net.classes_pad == self.cfg.num_classes else logits[:, :self.cfg.num_classes].contiguous()
        stats = K.xent_stats(real, labels)
        loss_rows, dlogits = K.xent_grad(real, labels, stats, grad_scale=1.0 / n)
        if net.classes_pad != self.cfg.num_classes:
            full = torch.zeros_like(logits)
            full[:, :self.cfg.num_classes] = dlogits
            dlogits = full
        net.backward(dlogits, stage_done=self._reduce_stage)
        if self.overlap:
            torch.cuda.current_stream().wait_stream(self.comm_stream)
        self.opt.step()
        return loss_rows.mean()

    @torch.no_grad()
    def predict(self, images):
        self.net.training = False
        return self.net.forward(images)[:, :self.cfg.num_classes]
