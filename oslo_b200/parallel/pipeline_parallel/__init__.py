from .partitioner import ModelPartitioner, PartitioningCostEstimator, PipeUnit
from .pipeline_parallel import PipelineParallel

__all__ = ["PipelineParallel", "ModelPartitioner", "PartitioningCostEstimator", "PipeUnit"]
