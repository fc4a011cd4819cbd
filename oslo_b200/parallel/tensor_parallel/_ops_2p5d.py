"""2.5-D (tesseract) tensor-parallel ops: a ``q x q`` SUMMA grid replicated ``d`` times along DEP.

Within a depth slice the maths is the 2-D algorithm over the 2.5-D ROW / COL groups.  Weights are identical
across depth (as in the reference, where depth is pure replication: oslo/.../_2p5d/_wrapper.py:241-262), but
here the batch is ALSO split over DEP, so the ``d`` slices do distinct work and weight gradients are summed
over DEP once per step by the wrapper.  Bias is ``[out/q]`` (out-block j), replicated along COL.

Parity: oslo/torch/nn/parallel/tensor_parallel/_2p5d/_ops.py:139-1094.
"""
from __future__ import annotations

from oslo_b200.distributed import ParallelMode

from . import _ops_nd as nd
from ._ops_2d import matmul_abt

ROW, COL, DEP = ParallelMode.TENSOR_2P5D_ROW, ParallelMode.TENSOR_2P5D_COL, ParallelMode.TENSOR_2P5D_DEP


def matmul_abt_2p5d(x, weight, pc):
    return matmul_abt(x, weight, pc, ROW, COL)


def all_gather_tensor_2p5d(t, dim, mode, pc):
    return nd.all_gather(t, dim, mode, pc)


def reduce_scatter_tensor_2p5d(t, dim, mode, pc):
    return nd.reduce_scatter(t, dim, mode, pc)


def gather_output_2p5d(t, pc):
    t = nd.gather_replicated(t, -1, ROW, pc)
    t = nd.gather_replicated(t, 0, COL, pc)
    return nd.gather_replicated(t, 0, DEP, pc)


def gather_batch_2p5d(ids, pc):
    return nd.gather_ids(ids, 0, COL, pc)
