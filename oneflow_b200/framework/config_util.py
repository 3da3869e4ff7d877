"""Process-wide resource switches (``flow.config`` style ``api_*`` setters; reference:
python/oneflow/framework/config_util.py:78-280).  The reference writes them into the session's Resource proto
before the first job is compiled; here they land in one type-checked dictionary (:func:`resource`).
``api_load_library`` really loads the library.  The collective-fusion switches describe behaviour that is fixed in this
framework (collectives are kernels over peer memory, gradients are reduced per flat bucket), so they are recorded and
reported but change nothing; scripts that set them keep working.
"""
import ctypes

_resource = {
    "load_library": [],
    "numa_aware_cuda_malloc_host": False,
    "reserved_device_mem_mbyte": 0,
    "enable_cudnn_fused_normalization_add_relu": True,
    "enable_cudnn_conv_heuristic_search_algo": True,
    "enable_fusion": True,
    "nccl_use_compute_stream": False,
    "disable_group_boxing_by_dst_parallel": False,
    "nccl_num_streams": 1,
    "nccl_fusion_threshold_mb": 16,
    "nccl_fusion_all_reduce_use_buffer": True,
    "nccl_fusion_all_reduce": True,
    "nccl_fusion_reduce_scatter": False,
    "nccl_fusion_all_gather": False,
    "nccl_fusion_reduce": True,
    "nccl_fusion_broadcast": True,
    "nccl_fusion_max_ops": 64,
    "nccl_enable_all_to_all": True,
    "nccl_enable_mixed_fusion": False,
}


def resource():
    """A copy of the current switches."""
    return dict(_resource)


def get(name, default=None):
    return _resource.get(name, default)


def _setter(name, typ, doc):
    def fn(val=True if typ is bool else None):
        if val is None:
            raise TypeError(f"{name}: a value is required")
        if not isinstance(val, typ) or (typ is int and isinstance(val, bool)):
            raise TypeError(f"{name}: expected {typ.__name__}, got {type(val).__name__}")
        _resource[name] = val
    fn.__name__ = "api_" + name
    fn.__doc__ = doc
    return fn


def api_load_library(val):
    """dlopen a shared library of extra kernels into the process and remember it."""
    ctypes.CDLL(str(val), mode=ctypes.RTLD_GLOBAL)
    _resource["load_library"].append(str(val))


api_numa_aware_cuda_malloc_host = _setter("numa_aware_cuda_malloc_host", bool, "Pin host memory on the GPU's NUMA node.")
api_reserved_device_mem_mbyte = _setter("reserved_device_mem_mbyte", int, "Device memory (MiB) the allocator leaves free.")
api_enable_cudnn_fused_normalization_add_relu = _setter(
    "enable_cudnn_fused_normalization_add_relu", bool, "Fused batch-norm + add + ReLU (always the path taken here).")
api_enable_cudnn_conv_heuristic_search_algo = _setter(
    "enable_cudnn_conv_heuristic_search_algo", bool, "Heuristic convolution algorithm choice (tile choice is static here).")
api_enable_fusion = _setter("enable_fusion", bool, "Fuse boxing collectives.")
api_nccl_use_compute_stream = _setter("nccl_use_compute_stream", bool, "Run collectives on the compute stream.")
api_disable_group_boxing_by_dst_parallel = _setter("disable_group_boxing_by_dst_parallel", bool,
                                                   "Do not group boxing ops by destination placement.")
api_nccl_num_streams = _setter("nccl_num_streams", int, "Number of collective streams.")
api_nccl_fusion_threshold_mb = _setter("nccl_fusion_threshold_mb", int, "Gradient bucket size in MiB.")
api_nccl_fusion_all_reduce_use_buffer = _setter("nccl_fusion_all_reduce_use_buffer", bool, "Fuse all-reduce through a flat buffer.")
api_nccl_fusion_all_reduce = _setter("nccl_fusion_all_reduce", bool, "Fuse all-reduce ops.")
api_nccl_fusion_reduce_scatter = _setter("nccl_fusion_reduce_scatter", bool, "Fuse reduce-scatter ops.")
api_nccl_fusion_all_gather = _setter("nccl_fusion_all_gather", bool, "Fuse all-gather ops.")
api_nccl_fusion_reduce = _setter("nccl_fusion_reduce", bool, "Fuse reduce ops.")
api_nccl_fusion_broadcast = _setter("nccl_fusion_broadcast", bool, "Fuse broadcast ops.")
api_nccl_fusion_max_ops = _setter("nccl_fusion_max_ops", int, "Most ops fused into one collective.")
api_nccl_enable_all_to_all = _setter("nccl_enable_all_to_all", bool, "Use all-to-all for S(i)->S(j) boxing.")
api_nccl_enable_mixed_fusion = _setter("nccl_enable_mixed_fusion", bool, "Fuse collectives of different kinds.")
