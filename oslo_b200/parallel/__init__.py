from .data_parallel import DistributedDataParallel, ShardingStrategy, ZeroRedundancyOptimizer
from .expert_parallel import ExpertParallel
from .tensor_parallel import TensorParallel

__all__ = ["TensorParallel", "ExpertParallel", "DistributedDataParallel", "ShardingStrategy", "ZeroRedundancyOptimizer"]
