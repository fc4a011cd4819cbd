"""Shared machinery of the fused optimizers: per (group, dtype) device tensor tables and dtype bucketing."""
from __future__ import annotations

from typing import Dict, List

import torch

from oslo_b200.ops import _lib
from oslo_b200.ops.multi_tensor import TensorTable

DT = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


class FusedOptimizerBase(torch.optim.Optimizer):
    def __init__(self, params, defaults, set_grad_none: bool = True):
        super().__init__(params, defaults)
        self.set_grad_none = set_grad_none
        self._tables: Dict[tuple, TensorTable] = {}

    def zero_grad(self, set_to_none: bool = None):
        super().zero_grad(set_to_none=self.set_grad_none if set_to_none is None else set_to_none)

    def _buckets(self, group) -> Dict[tuple, List[torch.nn.Parameter]]:
        out: Dict[tuple, List[torch.nn.Parameter]] = {}
        for p in group["params"]:
            if p.grad is None:
                continue
            if p.grad.is_sparse:
                raise RuntimeError(f"{type(self).__name__} does not support sparse gradients")
            out.setdefault((p.is_cuda and _lib.has_cuda_kernels() and p.dtype in DT and p.grad.dtype in DT, p.dtype, p.grad.dtype), []).append(p)
        return out

    def _table(self, key, cols) -> TensorTable:
        t = self._tables.get(key)
        n = len(next(c for c in cols if c is not None))
        if t is None or t.n != n:
            t = self._tables[key] = TensorTable(cols)
        else:
            t.update(cols)
        return t

    @staticmethod
    def _grads(ps):
        return [p.grad if p.grad.is_contiguous() else p.grad.contiguous() for p in ps]
