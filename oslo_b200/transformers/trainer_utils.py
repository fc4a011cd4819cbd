"""Names and factories the trainer shares with user scripts: learning-rate schedules, optimizer names, rank-filtered logging.

Parity: oslo/transformers/trainer_utils.py (``SchedulerType``, ``OptimizerNames``, ``log_dist``).  Here the two enums come
with the factories that act on them (:func:`get_scheduler`, :func:`create_optimizer`), so the trainer and a hand-written
loop build the same objects from the same strings.
"""
from __future__ import annotations

import enum
import logging
import math
import os
from typing import Iterable, Optional

import torch


class _StrEnum(str, enum.Enum):
    """Enum whose members compare equal to their string values and whose lookup failure lists the choices."""

    @classmethod
    def _missing_(cls, value):
        raise ValueError(f"{value!r} is not a valid {cls.__name__}; choose one of {[m.value for m in cls]}")

    def __str__(self):
        return self.value


class SchedulerType(_StrEnum):
    LINEAR = "linear"
    COSINE = "cosine"
    COSINE_WITH_RESTARTS = "cosine_with_restarts"
    POLYNOMIAL = "polynomial"
    CONSTANT = "constant"
    CONSTANT_WITH_WARMUP = "constant_with_warmup"


class OptimizerNames(_StrEnum):
    ADAM = "adam"
    ADAMW = "adamw"
    ADAGRAD = "adagrad"
    ADADELTA = "adadelta"
    ADAFACTOR = "adafactor"
    SGD = "sgd"
    NOVOGRAD = "novograd"
    LAMB = "lamb"
    CPU_ADAM = "cpu_adam"
    CPU_ADAGRAD = "cpu_adagrad"


class IntervalStrategy(_StrEnum):
    NO = "no"
    STEPS = "steps"
    EPOCH = "epoch"


def lr_factor(kind: SchedulerType, step: int, warmup: int, total: int, num_cycles: float = 0.5, power: float = 1.0,
              lr_end_ratio: float = 0.0) -> float:
    """Multiplier of the base learning rate at optimizer step ``step`` (0-based).  Warm-up is linear from 1/warmup to 1."""
    kind = SchedulerType(kind)
    if kind == SchedulerType.CONSTANT:
        return 1.0
    if warmup and step < warmup:
        return (step + 1) / warmup
    if kind == SchedulerType.CONSTANT_WITH_WARMUP:
        return 1.0
    frac = min(1.0, (step - warmup) / max(1, total - warmup))
    if kind == SchedulerType.LINEAR:
        return max(0.0, 1.0 - frac)
    if kind == SchedulerType.COSINE:
        return max(0.0, 0.5 * (1.0 + math.cos(math.pi * 2.0 * num_cycles * frac)))
    if kind == SchedulerType.COSINE_WITH_RESTARTS:
        if frac >= 1.0:
            return 0.0
        cycles = max(1.0, round(num_cycles)) if num_cycles >= 1 else 1.0
        return max(0.0, 0.5 * (1.0 + math.cos(math.pi * ((cycles * frac) % 1.0))))
    # polynomial decay to lr_end_ratio
    return lr_end_ratio + (1.0 - lr_end_ratio) * (1.0 - frac) ** power


def get_scheduler(name, optimizer, num_warmup_steps: int = 0, num_training_steps: int = 0, num_cycles: float = 0.5,
                  power: float = 1.0, lr_end_ratio: float = 0.0):
    kind = SchedulerType(name)
    if kind not in (SchedulerType.CONSTANT, SchedulerType.CONSTANT_WITH_WARMUP) and num_training_steps <= 0:
        raise ValueError(f"{kind.value} needs num_training_steps")
    return torch.optim.lr_scheduler.LambdaLR(
        optimizer, lambda s: lr_factor(kind, s, num_warmup_steps, num_training_steps, num_cycles, power, lr_end_ratio))


def create_optimizer(name, params: Iterable[torch.nn.Parameter], lr: float, weight_decay: float = 0.0, betas=(0.9, 0.999),
                     eps: float = 1e-8, max_grad_norm: float = 1.0, master_weights: bool = False, momentum: float = 0.0):
    """Build the optimizer ``name`` over ``params``: the fused multi-tensor kernels for the families that have one, the
    host-side SIMD optimizers for ``cpu_*``, stock PyTorch for Adadelta and Adafactor."""
    from oslo_b200 import optim

    kind = OptimizerNames(str(name).lower())
    params = list(params)
    if kind in (OptimizerNames.ADAM, OptimizerNames.ADAMW):
        return optim.FusedAdam(params, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, master_weights=master_weights)
    if kind == OptimizerNames.LAMB:
        return optim.FusedLamb(params, lr=lr, weight_decay=weight_decay, max_grad_norm=max_grad_norm)
    if kind == OptimizerNames.SGD:
        return optim.FusedSGD(params, lr=lr, weight_decay=weight_decay, momentum=momentum)
    if kind == OptimizerNames.ADAGRAD:
        return optim.FusedAdagrad(params, lr=lr, weight_decay=weight_decay)
    if kind == OptimizerNames.NOVOGRAD:
        return optim.FusedNovoGrad(params, lr=lr, weight_decay=weight_decay)
    if kind == OptimizerNames.CPU_ADAM:
        return optim.CPUAdam(params, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)
    if kind == OptimizerNames.CPU_ADAGRAD:
        return optim.CPUAdagrad(params, lr=lr, weight_decay=weight_decay)
    if kind == OptimizerNames.ADADELTA:
        return torch.optim.Adadelta(params, lr=lr, weight_decay=weight_decay)
    if kind == OptimizerNames.ADAFACTOR:
        return torch.optim.Adafactor(params, lr=lr, weight_decay=weight_decay)
    raise ValueError(kind)


_LEVELS = {"debug": logging.DEBUG, "info": logging.INFO, "warning": logging.WARNING, "error": logging.ERROR}


def log_dist(message: str, rank: int = 0, level=logging.INFO, logger: Optional[logging.Logger] = None) -> bool:
    """Log ``message`` on ``rank`` only (``-1``: every rank), prefixed with the rank.  Returns whether this rank logged."""
    me = int(os.environ.get("RANK", "0"))
    if rank != -1 and me != rank:
        return False
    if isinstance(level, str):
        level = _LEVELS[level.lower()]
    (logger or logging.getLogger("oslo_b200")).log(level, f"[Rank {me}] {message}")
    return True


__all__ = ["SchedulerType", "OptimizerNames", "IntervalStrategy", "lr_factor", "get_scheduler", "create_optimizer", "log_dist"]
