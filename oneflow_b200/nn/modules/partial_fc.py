"""Partial-FC class sampling for model-parallel softmax over very many classes
(reference: oneflow/user/kernels/partial_fc_sample_kernel.cu, op ``distributed_partial_fc_sample``).

The class-weight matrix [num_classes, dim] is split along dim 0 over the ranks. Each step a rank keeps the classes of
its shard that occur in the batch (positives) and fills up to ``num_sample`` local rows with random other classes
of its shard; labels are re-mapped into the sampled (concatenated over ranks) class space, labels owned by another
rank's shard map to that rank's sampled range."""
from __future__ import annotations

import torch
import torch.distributed as dist


def distributed_partial_fc_sample(weight, label, num_sample, group=None, generator=None):
    """weight: this rank's shard [classes_local, dim]; label: int64 [batch] global class ids (same on all ranks);
    num_sample: sampled classes per rank. Returns (mapped_label, sampled_label, sampled_weight)."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    classes_local = weight.shape[0]
    lo = rank * classes_local
    dev = weight.device
    num_sample = min(int(num_sample), classes_local)
    local = label[(label >= lo) & (label < lo + classes_local)] - lo
    pos = torch.unique(local)
    if pos.numel() > num_sample:
        raise ValueError(f"{pos.numel()} positive classes on this rank but only {num_sample} samples per rank")
    # random priorities, positives forced to the front, then take the first num_sample classes and sort them
    pri = torch.rand(classes_local, device=dev, generator=generator)
    pri[pos] = 2.0
    sampled = torch.topk(pri, num_sample).indices.sort().values
    sampled_weight = weight.index_select(0, sampled)
    # map every label to its position in the concatenated sampled class list (rank r owns [r * num_sample, ...))
    pos_of = torch.full((classes_local,), -1, dtype=torch.int64, device=dev)
    pos_of[sampled] = torch.arange(num_sample, device=dev) + rank * num_sample
    mapped = torch.full_like(label, -1)
    mine = (label >= lo) & (label < lo + classes_local)
    mapped[mine] = pos_of[label[mine] - lo]
    if world > 1:
        dist.all_reduce(mapped, op=dist.ReduceOp.MAX, group=group)     # every label is owned by exactly one rank
    return mapped, sampled + lo, sampled_weight
