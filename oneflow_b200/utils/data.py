"""``flow.utils.data``: torch's DataLoader machinery (worker processes, shared-memory tensor passing,
samplers, DistributedSampler) under the flow names. Reference: python/oneflow/utils/data/*."""
from torch.utils.data import *  # noqa: F401,F403
from torch.utils.data import (BatchSampler, DataLoader, Dataset, IterableDataset, RandomSampler, Sampler,  # noqa: F401
                              SequentialSampler, Subset, TensorDataset, random_split)
from torch.utils.data.distributed import DistributedSampler  # noqa: F401
from torch.utils.data import distributed  # noqa: F401
