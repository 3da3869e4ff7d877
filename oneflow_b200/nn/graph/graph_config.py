"""``graph.config``: the knobs of nn.Graph (reference: python/oneflow/nn/graph/graph_config.py:50-470).
Each setter records the option; nn.Graph reads them when it prepares its step function."""
from __future__ import annotations

import warnings

import torch

_warned = set()


def _no_effect(name, why):
    """Some switches of the reference steer compiler passes that have no counterpart in this runtime. They are accepted
    (scripts keep running) and say so once per process instead of silently doing nothing."""
    if name not in _warned:
        _warned.add(name)
        warnings.warn(f"nn.Graph config.{name} is accepted but changes nothing here: {why}", stacklevel=3)


class GraphConfig:
    def __init__(self):
        self.training = False
        self.amp_enabled = False
        self.amp_dtype = torch.float16
        self.zero_stage = 0
        self.zero_shard_min_size = 1024
        self.zero_shard_restore_level = 1
        self.grad_acc_steps = 1
        self.outputs_buffer_size = 2
        self.fuse_model_update_ops = False
        self.fuse_add_to_output = False
        self.fuse_cast_scale = False
        self.cudnn_conv_heuristic_search = True
        self.straighten_algorithm = "MemoryFirst"
        self.compress_memory = False
        self.auto_parallel = False
        self.auto_memory = None
        self.multi_tensor_update = False
        self.fused_model_update_cast = False
        self.cuda_graph = False
        self.debug_level = -1
        self.extra = {}

    # --- mixed precision
    def enable_amp(self, mode: bool = True, *, dtype=torch.float16):
        self.amp_enabled, self.amp_dtype = bool(mode), dtype

    # --- ZeRO
    def enable_zero(self, mode: bool = True, *, stage: int = 2, shard_min_size: int = 1024, shard_restore_level: int = 1):
        self.zero_stage = int(stage) if mode else 0
        self.zero_shard_min_size = shard_min_size
        self.zero_shard_restore_level = shard_restore_level

    def set_zero_redundancy_optimizer_mode(self, mode="distributed_split"):
        self.extra["zero_mode"] = mode

    # --- gradient accumulation
    def set_gradient_accumulation_steps(self, value: int):
        if value < 1:
            raise ValueError("gradient accumulation steps must be >= 1")
        self.grad_acc_steps = int(value)

    def set_outputs_buffer_size(self, value: int = 2):
        self.outputs_buffer_size = int(value)

    # --- fusion / scheduling hints (the engine already fuses these; the flags are recorded for introspection)
    def allow_fuse_model_update_ops(self, mode: bool = True):
        self.fuse_model_update_ops = bool(mode)

    def allow_fuse_add_to_output(self, mode: bool = True):
        self.fuse_add_to_output = bool(mode)

    def allow_fuse_cast_scale(self, mode: bool = True):
        self.fuse_cast_scale = bool(mode)

    def enable_cudnn_conv_heuristic_search_algo(self, mode: bool = True):
        self.cudnn_conv_heuristic_search = bool(mode)
        _no_effect("enable_cudnn_conv_heuristic_search_algo", "convolutions run the in-tree implicit-GEMM kernels or PyTorch's, not a cuDNN algorithm search")

    def enable_straighten_algorithm(self, mode: str = "MemoryFirst"):
        if mode not in ("Disable", "SpeedFirst", "MemoryFirst", "OverlapCpuGpu", "DelayShortGpu"):
            raise ValueError(f"unknown straighten mode {mode}")
        self.straighten_algorithm = mode
        _no_effect("enable_straighten_algorithm", "kernels launch in program order on CUDA streams, there is no task graph to reorder")

    def enable_compress_memory(self, mode: bool = True):
        self.compress_memory = bool(mode)
        if mode:
            _no_effect("enable_compress_memory", "memory comes from the caching allocator, there is no static memory plan to compress")

    def enable_choose_best_memory_allocation(self, mode: bool = True):
        self.extra["best_memory_allocation"] = bool(mode)
        if mode:
            _no_effect("enable_choose_best_memory_allocation", "there is no static memory plan")

    def enable_auto_parallel(self, mode: bool = True):
        self.auto_parallel = bool(mode)

    def enable_auto_parallel_ignore_user_sbp_config(self, mode: bool = True):
        self.extra["auto_parallel_ignore_user_sbp"] = bool(mode)

    def set_auto_parallel_computation_cost_ratio(self, ratio):
        self.extra["auto_parallel_computation_cost_ratio"] = ratio

    def set_auto_parallel_wait_time(self, cost):
        self.extra["auto_parallel_wait_time"] = cost

    def enable_auto_parallel_trunk_algo(self, mode: bool = True):
        self.extra["auto_parallel_trunk_algo"] = bool(mode)

    def enable_auto_parallel_sbp_collector(self, mode: bool = True):
        self.extra["auto_parallel_sbp_collector"] = bool(mode)

    def enable_auto_memory(self, mode="AdaptiveMemory"):
        self.auto_memory = mode
        _no_effect("enable_auto_memory", "use GraphModule.activation_checkpointing per block to trade compute for memory")

    def enable_multi_tensor_update(self, mode: bool = True):
        self.multi_tensor_update = bool(mode)

    def enable_fused_model_update_cast(self, mode: bool = True):
        # always in effect for bf16 parameters: the flat optimizer writes the low-precision copy in the update kernel
        self.fused_model_update_cast = bool(mode)

    def enable_cuda_graph(self, mode: bool = True):
        """Capture the whole step in a CUDA graph after the first call (static shapes, CUDA tensors)."""
        self.cuda_graph = bool(mode)

    def _as_dict(self):
        return {k: (str(v) if isinstance(v, torch.dtype) else v) for k, v in vars(self).items() if not k.startswith("_")}

    @property
    def proto(self):
        """The job configuration as a plain dict (the reference holds a JobConfigProto); nn.Graph adds the optimizer
        entries when it compiles."""
        return getattr(self, "_proto", None) or self._as_dict()

    def __repr__(self):
        return f"GraphConfig({ {k: v for k, v in self.__dict__.items() if k != 'extra'} })"
