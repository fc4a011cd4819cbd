"""Optimizers (parity: oslo/torch/optim/__init__.py:1-6)."""
from .cpu_adam import CPUAdagrad, CPUAdam
from .fused_adagrad import FusedAdagrad
from .fused_adam import FusedAdam
from .fused_lamb import FusedLamb, FusedMixedPrecisionLamb
from .fused_novograd import FusedNovoGrad
from .fused_sgd import FusedSGD
from .loss_scaler import DynamicLossScaler

__all__ = ["FusedAdam", "FusedSGD", "FusedAdagrad", "FusedLamb", "FusedMixedPrecisionLamb", "FusedNovoGrad", "CPUAdam",
           "CPUAdagrad", "DynamicLossScaler"]
