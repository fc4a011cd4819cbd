"""2-D (SUMMA) tensor-parallel ops on a ``q x q`` grid; rank ``(i, j)`` = (rank in COL group, rank in ROW group).

Layouts (identical to the reference so checkpoints interchange): activations ``[b/q (i), s, h/q (j)]``;
``Linear2D`` weight ``W[out/q (i), in/q (j)]``, bias ``[out/q^2]`` = out-block ``j`` split again over ``i``.

``C_ij = sum_k X_ik W_jk^T`` is evaluated as *gather the weight column, multiply, reduce-scatter the row*:

    W_:j = all_gather(W_ij over COL)            [out, in/q]
    P    = X_ij W_:j^T                          [b/q, s, out]   (partial over j)
    C_ij = reduce_scatter(P over ROW, last dim) [b/q, s, out/q]

i.e. 2 collectives per product instead of the reference's 2q broadcasts / reduces with a host-side loop
(oslo/torch/nn/parallel/tensor_parallel/_2d/_ops.py:283-309,437-464,601-625); autograd yields the adjoints
(dX: all-gather dC over ROW; dW: reduce-scatter over COL).
"""
from __future__ import annotations

from oslo_b200.distributed import ParallelMode
from oslo_b200.ops.gemm import linear

from . import _ops_nd as nd

ROW, COL = ParallelMode.TENSOR_2D_ROW, ParallelMode.TENSOR_2D_COL


def matmul_abt(x, weight, pc, row_mode, col_mode):
    w_col = nd.all_gather(weight, 0, col_mode, pc)
    partial = linear(x, w_col)
    return nd.reduce_scatter(partial, -1, row_mode, pc)


def matmul_abt_2d(x, weight, pc):
    return matmul_abt(x, weight, pc, ROW, COL)


def gather_bias_2d(bias, pc):
    """``[out/q^2] -> [out/q]`` (out-block j): all-gather over COL, reduce-scatter in backward."""
    return nd.all_gather(bias, 0, COL, pc)


def add_bias_2d(out, bias, pc):
    return out + gather_bias_2d(bias, pc)


def all_gather_tensor_2d(t, dim, mode, pc):
    return nd.all_gather(t, dim, mode, pc)


def reduce_scatter_tensor_2d(t, dim, mode, pc):
    return nd.reduce_scatter(t, dim, mode, pc)


def gather_output_2d(t, pc):
    """Full ``[b, s, out]`` on every rank (for heads whose consumers are replicated)."""
    t = nd.gather_replicated(t, -1, ROW, pc)
    return nd.gather_replicated(t, 0, COL, pc)


def gather_batch_2d(ids, pc):
    return nd.gather_ids(ids, 0, COL, pc)


def split_batch_2d(t, dim, pc):
    from oslo_b200.distributed import comm

    return comm.scatter(t, dim=dim, parallel_context=pc, parallel_mode=COL)
