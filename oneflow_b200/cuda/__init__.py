"""``flow.cuda``: device management, synchronisation, seeds and memory statistics (torch.cuda)."""
from torch.cuda import *  # noqa: F401,F403
from torch.cuda import (current_device, current_stream, device_count, empty_cache, is_available, manual_seed,  # noqa: F401
                        manual_seed_all, max_memory_allocated, memory_allocated, memory_reserved, set_device, synchronize)
