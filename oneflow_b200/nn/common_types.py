"""``flow.nn.common_types``: the size / tuple type aliases used in layer signatures; identical to torch's."""
from torch.nn.common_types import *  # noqa: F401,F403
from torch.nn.common_types import (_size_1_t, _size_2_t, _size_3_t, _size_4_t, _size_5_t, _size_6_t, _size_any_t,  # noqa: F401
                                   _ratio_2_t, _ratio_3_t, _ratio_any_t, _tensor_list_t, _maybe_indices_t,
                                   _scalar_or_tuple_1_t, _scalar_or_tuple_2_t, _scalar_or_tuple_3_t, _scalar_or_tuple_4_t,
                                   _scalar_or_tuple_5_t, _scalar_or_tuple_6_t, _scalar_or_tuple_any_t, _size_any_opt_t,
                                   _size_2_opt_t, _size_3_opt_t)
