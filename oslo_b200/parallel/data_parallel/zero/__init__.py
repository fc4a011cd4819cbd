from .optim import ZeroRedundancyOptimizer

__all__ = ["ZeroRedundancyOptimizer"]
