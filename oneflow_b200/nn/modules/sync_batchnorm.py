"""SyncBatchNorm: batch statistics over the whole data-parallel group
(reference: python/oneflow/nn/modules/batchnorm.py SyncBatchNorm and the kernels batch_norm_stats /
batch_norm_gather_stats_with_counts / batch_norm_elemt / batch_norm_backward_reduce / batch_norm_backward_elemt).
Forward exchanges per-channel (count, sum, sum of squares); backward exchanges (sum dy, sum dy * xhat): two small
all-reduces per layer and direction."""
from __future__ import annotations

import torch
import torch.distributed as dist


class _SyncBNFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, eps, group):
        c = x.shape[1]
        dims = [0] + list(range(2, x.dim()))
        xf = x.float()
        stats = torch.cat([xf.sum(dims), (xf * xf).sum(dims), torch.full((1,), float(x.numel() // c), device=x.device)])
        if dist.is_initialized() and dist.get_world_size(group) > 1:
            dist.all_reduce(stats, group=group)
        n = stats[-1]
        mean = stats[:c] / n
        var = (stats[c:2 * c] / n - mean * mean).clamp_min(0)
        rstd = torch.rsqrt(var + eps)
        shape = [1, c] + [1] * (x.dim() - 2)
        xhat = (xf - mean.view(shape)) * rstd.view(shape)
        y = xhat * weight.float().view(shape) + bias.float().view(shape)
        ctx.save_for_backward(xhat, weight, rstd, n)
        ctx.group, ctx.dims, ctx.shape = group, dims, shape
        ctx.mark_non_differentiable(mean, var)
        return y.to(x.dtype), mean, var

    @staticmethod
    def backward(ctx, dy, _dm, _dv):
        xhat, weight, rstd, n = ctx.saved_tensors
        c = xhat.shape[1]
        g = dy.float()
        local = torch.cat([g.sum(ctx.dims), (g * xhat).sum(ctx.dims)])
        total = local.clone()
        if dist.is_initialized() and dist.get_world_size(ctx.group) > 1:
            dist.all_reduce(total, group=ctx.group)
        s1, s2 = total[:c].view(ctx.shape), total[c:].view(ctx.shape)
        dx = weight.float().view(ctx.shape) * rstd.view(ctx.shape) * (g - s1 / n - xhat * s2 / n)
        return dx.to(dy.dtype), local[c:].to(weight.dtype), local[:c].to(weight.dtype), None, None


class SyncBatchNorm(torch.nn.modules.batchnorm._BatchNorm):
    def __init__(self, num_features, eps=1e-5, momentum=0.1, affine=True, track_running_stats=True, process_group=None,
                 device=None, dtype=None):
        super().__init__(num_features, eps, momentum, affine, track_running_stats, device=device, dtype=dtype)
        self.process_group = process_group

    def _check_input_dim(self, input):
        if input.dim() < 2:
            raise ValueError(f"expected at least 2D input (got {input.dim()}D input)")

    def forward(self, x):
        self._check_input_dim(x)
        if not self.training and self.track_running_stats:
            return torch.nn.functional.batch_norm(x, self.running_mean, self.running_var, self.weight, self.bias, False, 0.0, self.eps)
        w = self.weight if self.affine else torch.ones(self.num_features, device=x.device)
        b = self.bias if self.affine else torch.zeros(self.num_features, device=x.device)
        y, mean, var = _SyncBNFn.apply(x, w, b, self.eps, self.process_group)
        if self.track_running_stats:
            with torch.no_grad():
                m = self.momentum if self.momentum is not None else 0.1
                world = dist.get_world_size(self.process_group) if dist.is_initialized() else 1
                count = x.numel() // x.shape[1] * world
                self.running_mean.mul_(1 - m).add_(mean.to(self.running_mean.dtype), alpha=m)
                self.running_var.mul_(1 - m).add_((var * count / max(count - 1, 1)).to(self.running_var.dtype), alpha=m)
                self.num_batches_tracked += 1
        return y

    @classmethod
    def convert_sync_batchnorm(cls, module, process_group=None):
        out = module
        if isinstance(module, torch.nn.modules.batchnorm._BatchNorm) and not isinstance(module, cls):
            out = cls(module.num_features, module.eps, module.momentum, module.affine, module.track_running_stats, process_group)
            if module.affine:
                out.weight, out.bias = module.weight, module.bias
            out.running_mean, out.running_var, out.num_batches_tracked = module.running_mean, module.running_var, module.num_batches_tracked
        for name, child in module.named_children():
            out.add_module(name, cls.convert_sync_batchnorm(child, process_group))
        return out
