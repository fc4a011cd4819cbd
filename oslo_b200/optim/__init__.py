from .fused_adam import FusedAdam

__all__ = ["FusedAdam"]
