"""Splits a model's sequence of pipeline units into ``pp`` contiguous stages of balanced cost.

Cost of a unit = ``alpha * normalised parameter count + (1 - alpha) * normalised forward time`` where ``alpha`` is
the wrapper's ``memory_computation_balance`` (1.0 = balance memory only), as in the reference's
``PartitioningCostEstimator`` (oslo/torch/nn/parallel/pipeline_parallel/_cost_estimator.py:12-144).  The split is the
optimal contiguous partition minimising the largest stage cost (dynamic programme over prefix sums) — the same
objective the reference's ``ModelPartitioner`` pursues over its module tree (_model_partitioner.py:79-284).
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

import torch
import torch.nn as nn


@dataclass
class PipeUnit:
    """One indivisible step of a model's forward: ``fn(state) -> state`` using ``modules``."""

    name: str
    modules: List[nn.Module]
    fn: Callable[[dict], dict]
    flops_hint: float = 0.0

    def parameters(self):
        seen = set()
        for m in self.modules:
            for p in m.parameters():
                if id(p) not in seen:
                    seen.add(id(p))
                    yield p


class PartitioningCostEstimator:
    def __init__(self, units: Sequence[PipeUnit], alpha: float = 1.0, measure: Optional[Callable[[PipeUnit], float]] = None):
        self.units, self.alpha, self.measure = list(units), float(alpha), measure

    def costs(self) -> List[float]:
        mem = [float(sum(p.numel() for p in u.parameters())) for u in self.units]
        if self.alpha >= 1.0:
            comp = [0.0] * len(self.units)
        elif self.measure is not None:
            comp = [self.measure(u) for u in self.units]
        else:
            comp = [u.flops_hint or m for u, m in zip(self.units, mem)]
        norm = lambda v: [x / (sum(v) or 1.0) for x in v]
        mem, comp = norm(mem), norm(comp)
        return [self.alpha * m + (1.0 - self.alpha) * c for m, c in zip(mem, comp)]


class ModelPartitioner:
    def __init__(self, units: Sequence[PipeUnit], num_stages: int, memory_computation_balance: float = 1.0):
        if num_stages > len(units):
            raise ValueError(f"cannot split {len(units)} units into {num_stages} stages")
        self.units, self.num_stages = list(units), num_stages
        self.costs = PartitioningCostEstimator(units, memory_computation_balance).costs()

    def partition(self) -> List[range]:
        """Contiguous unit ranges per stage minimising the maximum stage cost."""
        n, k = len(self.units), self.num_stages
        prefix = [0.0]
        for c in self.costs:
            prefix.append(prefix[-1] + c)
        seg = lambda i, j: prefix[j] - prefix[i]
        INF = float("inf")
        best = [[INF] * (n + 1) for _ in range(k + 1)]
        cut = [[0] * (n + 1) for _ in range(k + 1)]
        best[0][0] = 0.0
        for s in range(1, k + 1):
            for j in range(s, n - (k - s) + 1):
                for i in range(s - 1, j):
                    v = max(best[s - 1][i], seg(i, j))
                    if v < best[s][j] - 1e-15:
                        best[s][j], cut[s][j] = v, i
        bounds, j = [], n
        for s in range(k, 0, -1):
            i = cut[s][j]
            bounds.append(range(i, j))
            j = i
        return list(reversed(bounds))

    def stage_costs(self) -> List[float]:
        return [sum(self.costs[i] for i in r) for r in self.partition()]


def sequential_units(module: nn.Module) -> List[PipeUnit]:
    """Pipeline units of an ``nn.Sequential`` (state key ``hidden``)."""
    units = []
    for name, child in module.named_children():
        def fn(state, child=child):
            state["hidden"] = child(state["hidden"])
            return state

        units.append(PipeUnit(name, [child], fn))
    return units
