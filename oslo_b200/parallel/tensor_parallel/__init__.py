from .tensor_parallel import TensorParallel

__all__ = ["TensorParallel"]
