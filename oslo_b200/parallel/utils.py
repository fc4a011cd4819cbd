"""Wrapper registry and the ``parallelize`` step behind :func:`oslo_b200.ready`.

Parity: oslo/torch/nn/parallel/utils.py:59-130.
"""
from __future__ import annotations

from typing import Dict

import torch
import torch.nn as nn

from oslo_b200.distributed import ParallelMode


class ParallelWrapper(nn.Module):
    """Base of TensorParallel / PipelineParallel / ExpertParallel / DistributedDataParallel wrappers."""

    parallelism_priority = 0

    def parallelize(self):
        raise NotImplementedError

    def deparallelize(self):
        raise NotImplementedError


def is_wrapper(obj) -> bool:
    return isinstance(obj, ParallelWrapper)


def unwrap_parallel(module):
    while is_wrapper(module):
        module = module.module
    return module


def get_parallel_context(module, parallel_context=None):
    if parallel_context is not None:
        return parallel_context
    from oslo_b200.distributed import ParallelContext

    pc = getattr(unwrap_parallel(module), "parallel_context", None) or ParallelContext.get_context()
    if pc is None:
        raise RuntimeError("no ParallelContext: create one with ParallelContext.from_torch(...) first")
    return pc


def add_wrapper(module: nn.Module, mode: ParallelMode, wrapper: ParallelWrapper):
    """Record ``wrapper`` on the (unwrapped) module so ``ready`` can run it later."""
    base = unwrap_parallel(module)
    if not hasattr(base, "oslo_wrappers"):
        base.oslo_wrappers = {}
    base.oslo_wrappers[mode] = wrapper


def parallelize(module: nn.Module, parallel_context):
    """Run every registered wrapper in priority order, rebind ``forward`` and place tensors on this rank's device."""
    base = unwrap_parallel(module)
    wrappers: Dict[ParallelMode, ParallelWrapper] = getattr(base, "oslo_wrappers", {})
    for wrapper in sorted(wrappers.values(), key=lambda w: w.parallelism_priority):
        if getattr(wrapper, "_parallelized", False):
            continue
        wrapper.parallelize()
        wrapper._parallelized = True
        base.oslo_forward_chain = getattr(base, "oslo_forward_chain", []) + [wrapper]
    device = parallel_context.device
    to_device(base, device)
    return module


def to_device(module: nn.Module, device):
    """Move parameters and buffers in place (keeps Parameter identity, so tied weights stay tied)."""
    if device.type == "cpu":
        return
    seen = set()
    for m in module.modules():
        for name, p in list(m._parameters.items()):
            if p is None or id(p) in seen:
                continue
            seen.add(id(p))
            if p.device != device:
                p.data = p.data.to(device)
                if p.grad is not None:
                    p.grad.data = p.grad.data.to(device)
        for name, b in list(m._buffers.items()):
            if b is not None and b.device != device:
                m._buffers[name] = b.to(device)


def allocate_params(module, parallel_context):
    to_device(unwrap_parallel(module), parallel_context.device)
