from .data_parallel import DistributedDataParallel, ShardingStrategy, ZeroRedundancyOptimizer
from .tensor_parallel import TensorParallel

__all__ = ["TensorParallel", "DistributedDataParallel", "ShardingStrategy", "ZeroRedundancyOptimizer"]
