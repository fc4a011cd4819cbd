from .data_parallel import DistributedDataParallel, ShardingStrategy, ZeroRedundancyOptimizer
from .expert_parallel import ExpertParallel
from .pipeline_parallel import PipelineParallel
from .tensor_parallel import TensorParallel

__all__ = ["TensorParallel", "PipelineParallel", "ExpertParallel", "DistributedDataParallel", "ShardingStrategy",
           "ZeroRedundancyOptimizer"]
