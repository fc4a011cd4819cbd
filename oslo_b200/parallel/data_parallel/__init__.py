from .data_parallel import DistributedDataParallel, ShardingStrategy, _DistributedDataParallel
from .zero import ZeroRedundancyOptimizer

__all__ = ["DistributedDataParallel", "ShardingStrategy", "ZeroRedundancyOptimizer"]
