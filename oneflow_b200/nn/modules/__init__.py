from .fused_mlp import FusedMLP, fused_linear_act  # noqa: F401
