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

On CUDA, once ``symm.enable(pc, <ROW mode>, ...)`` has built the row group's symmetric workspace, the product and the
activation-sized reduce-scatter are ONE kernel (``oslo_gemm_rs`` with the columns scattered): the epilogue of a tile of
another rank's feature block TMA-stores it into that rank's memory, the tiles of the own block are computed last and
fold the received partials in.  The weight all-gather stays a library collective: it does not depend on the
activations, so it is small and is shared by every micro-batch.
"""
from __future__ import annotations

import torch

from oslo_b200.distributed import ParallelMode
from oslo_b200.ops.gemm import linear

from . import _ops_nd as nd

ROW, COL = ParallelMode.TENSOR_2D_ROW, ParallelMode.TENSOR_2D_COL


class _LinearFeatureRS(torch.autograd.Function):
    """``reduce_scatter_features(x W^T)`` as one fused kernel; backward = all-gather(dC over ROW) then two GEMMs."""

    @staticmethod
    def forward(ctx, x, w_col, pc, row_mode):
        from oslo_b200.ops import fused_collectives as fc

        ctx.pc, ctx.row_mode, ctx.shape = pc, row_mode, x.shape
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        ctx.save_for_backward(x2, w_col)
        out = fc.gemm_rs_features(x2, w_col, row_mode)
        return out.view(*x.shape[:-1], out.shape[-1])

    @staticmethod
    def backward(ctx, g):
        from oslo_b200.distributed import comm
        from oslo_b200.ops.gemm import matmul_nt

        x2, w_col = ctx.saved_tensors
        g2 = g.reshape(-1, g.shape[-1]).contiguous()
        g_full = comm.all_gather(g2, dim=-1, parallel_context=ctx.pc, parallel_mode=ctx.row_mode)
        gx = matmul_nt(g_full, w_col.t()).view(ctx.shape) if ctx.needs_input_grad[0] else None
        gw = matmul_nt(g_full.t(), x2.t()) if ctx.needs_input_grad[1] else None
        return gx, gw, None, None


def matmul_abt(x, weight, pc, row_mode, col_mode):
    w_col = nd.all_gather(weight, 0, col_mode, pc)
    if x.is_cuda and pc.get_world_size(row_mode) > 1:
        from oslo_b200.ops import fused_collectives as fc

        x2 = x.reshape(-1, x.shape[-1])
        if fc.feature_rs_available(x2, w_col, row_mode):
            return _LinearFeatureRS.apply(x, w_col, pc, row_mode)
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
