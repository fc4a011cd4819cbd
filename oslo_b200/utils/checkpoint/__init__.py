from .activation_checkpointing import (
    ActivationCheckpointing,
    CheckpointFunction,
    CheckpointPartitioner,
    CudaRNGStatesTracker,
    checkpoint,
)

__all__ = ["ActivationCheckpointing", "CheckpointFunction", "CheckpointPartitioner", "CudaRNGStatesTracker", "checkpoint"]
