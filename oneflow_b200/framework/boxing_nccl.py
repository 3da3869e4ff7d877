"""``flow.boxing.nccl``: collective-fusion switches (reference: python/oneflow/boxing/nccl/__init__.py:16-41)."""
from .config_util import api_disable_group_boxing_by_dst_parallel as disable_group_boxing_by_dst_parallel  # noqa: F401
from .config_util import api_nccl_enable_all_to_all as enable_all_to_all  # noqa: F401
from .config_util import api_nccl_enable_mixed_fusion as allow_fuse_mixed_ops  # noqa: F401
from .config_util import api_nccl_fusion_all_gather as allow_fuse_all_gather  # noqa: F401
from .config_util import api_nccl_fusion_all_reduce as allow_fuse_all_reduce  # noqa: F401
from .config_util import api_nccl_fusion_all_reduce_use_buffer as enable_use_buffer_to_fuse_all_reduce  # noqa: F401
from .config_util import api_nccl_fusion_broadcast as allow_fuse_broadcast  # noqa: F401
from .config_util import api_nccl_fusion_max_ops as set_fusion_max_ops_num  # noqa: F401
from .config_util import api_nccl_fusion_reduce as allow_fuse_reduce  # noqa: F401
from .config_util import api_nccl_fusion_reduce_scatter as allow_fuse_reduce_scatter  # noqa: F401
from .config_util import api_nccl_fusion_threshold_mb as set_fusion_threshold_mbytes  # noqa: F401
from .config_util import api_nccl_num_streams as set_stream_num  # noqa: F401
from .config_util import api_nccl_use_compute_stream as enable_use_compute_stream  # noqa: F401
