"""Autograd-aware communication ops for 1-D (Megatron) tensor parallelism.

Besides the five classic conjugate pairs of the reference
(``oslo/torch/nn/parallel/tensor_parallel/_1d/_ops.py:17-157``) this file holds
the two *sequence-parallel* linears the reference lacks:

* ``ag_linear``   all-gather(tokens) -> GEMM      (column-parallel; backward: GEMM -> reduce-scatter)
* ``linear_rs``   GEMM -> reduce-scatter(tokens)  (row-parallel;    backward: all-gather -> GEMM)

On CUDA both run as ONE fused kernel over NVLink peer memory
(:mod:`oslo_b200.ops.fused_collectives`); elsewhere they are the equivalent
collective + matmul composition, which is also the correctness oracle.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from oslo_b200.distributed import ParallelMode
from oslo_b200.distributed import comm

_MODE = ParallelMode.TENSOR_1D


class _Broadcast1D(torch.autograd.Function):
    """identity forward, all-reduce backward (input of a column-parallel linear)."""

    @staticmethod
    def forward(ctx, x, pc):
        ctx.pc = pc
        return x

    @staticmethod
    def backward(ctx, g):
        return comm.all_reduce(g.contiguous(), parallel_context=ctx.pc, parallel_mode=_MODE), None


class _Reduce1D(torch.autograd.Function):
    """all-reduce forward, identity backward (output of a row-parallel linear)."""

    @staticmethod
    def forward(ctx, x, pc):
        return comm.all_reduce(x.contiguous(), parallel_context=pc, parallel_mode=_MODE)

    @staticmethod
    def backward(ctx, g):
        return g, None


class _Gather1D(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dim, pc):
        ctx.pc, ctx.dim = pc, dim
        return comm.all_gather(x, dim=dim, parallel_context=pc, parallel_mode=_MODE)

    @staticmethod
    def backward(ctx, g):
        return comm.scatter(g, dim=ctx.dim, parallel_context=ctx.pc, parallel_mode=_MODE), None, None


class _Scatter1D(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dim, pc):
        ctx.pc, ctx.dim = pc, dim
        return comm.scatter(x, dim=dim, parallel_context=pc, parallel_mode=_MODE)

    @staticmethod
    def backward(ctx, g):
        return comm.all_gather(g, dim=ctx.dim, parallel_context=ctx.pc, parallel_mode=_MODE), None, None


class _ReduceScatter1D(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dim, pc):
        ctx.pc, ctx.dim = pc, dim
        return comm.reduce_scatter(x, dim=dim, parallel_context=pc, parallel_mode=_MODE)

    @staticmethod
    def backward(ctx, g):
        return comm.all_gather(g, dim=ctx.dim, parallel_context=ctx.pc, parallel_mode=_MODE), None, None


class _GatherSeq1D(torch.autograd.Function):
    """all-gather forward, reduce-scatter backward (entering a tensor-parallel region under SP)."""

    @staticmethod
    def forward(ctx, x, dim, pc):
        ctx.pc, ctx.dim = pc, dim
        return comm.all_gather(x, dim=dim, parallel_context=pc, parallel_mode=_MODE)

    @staticmethod
    def backward(ctx, g):
        return comm.reduce_scatter(g, dim=ctx.dim, parallel_context=ctx.pc, parallel_mode=_MODE), None, None


def broadcast_tensor_1d(x, parallel_context):
    return _Broadcast1D.apply(x, parallel_context)


def reduce_tensor_1d(x, parallel_context):
    return _Reduce1D.apply(x, parallel_context)


def gather_tensor_1d(x, dim, parallel_context):
    return _Gather1D.apply(x, dim, parallel_context)


def scatter_tensor_1d(x, dim, parallel_context):
    return _Scatter1D.apply(x, dim, parallel_context)


def reduce_scatter_tensor_1d(x, dim, parallel_context):
    return _ReduceScatter1D.apply(x, dim, parallel_context)


def gather_sequence_1d(x, dim, parallel_context):
    return _GatherSeq1D.apply(x, dim, parallel_context)


# ----------------------------------------------------------- sequence-parallel linears
def _use_fused(x, weight, kind) -> bool:
    from oslo_b200.ops import fused_collectives as fc

    return fc.available(x, weight, kind)


class _AGLinear(torch.autograd.Function):
    """y_full = all_gather(x_shard, dim 0) @ W^T.  x_shard: [T/tp, K] (tokens flattened)."""

    @staticmethod
    def forward(ctx, x, weight, pc):
        ctx.pc = pc
        if _use_fused(x, weight, "ag"):
            from oslo_b200.ops import fused_collectives as fc

            y, x_full = fc.ag_gemm(x, weight, pc)
        else:
            from oslo_b200.ops.gemm import matmul_nt

            x_full = comm.all_gather(x, dim=0, parallel_context=pc, parallel_mode=_MODE)
            y = matmul_nt(x_full, weight)
        ctx.save_for_backward(x_full, weight)
        return y

    @staticmethod
    def backward(ctx, gy):
        x_full, weight = ctx.saved_tensors
        pc = ctx.pc
        gy = gy.contiguous()
        gx = gw = None
        if ctx.needs_input_grad[0]:
            if _use_fused(gy, weight.t(), "rs"):
                from oslo_b200.ops import fused_collectives as fc

                gx = fc.gemm_rs(gy, weight.t(), pc)
            else:
                from oslo_b200.ops.gemm import matmul_nt

                gx_full = matmul_nt(gy, weight.t())
                gx = comm.reduce_scatter(gx_full, dim=0, parallel_context=pc, parallel_mode=_MODE)
        if ctx.needs_input_grad[1]:
            from oslo_b200.ops.gemm import matmul_nt

            gw = matmul_nt(gy.t(), x_full.t())
        return gx, gw, None


class _LinearRS(torch.autograd.Function):
    """y_shard = reduce_scatter(x @ W^T, dim 0).  x: [T, K/tp] -> y: [T/tp, N]."""

    @staticmethod
    def forward(ctx, x, weight, pc):
        ctx.pc = pc
        ctx.save_for_backward(x, weight)
        if _use_fused(x, weight, "rs"):
            from oslo_b200.ops import fused_collectives as fc

            return fc.gemm_rs(x, weight, pc)
        from oslo_b200.ops.gemm import matmul_nt

        y = matmul_nt(x, weight)
        return comm.reduce_scatter(y, dim=0, parallel_context=pc, parallel_mode=_MODE)

    @staticmethod
    def backward(ctx, gy):
        x, weight = ctx.saved_tensors
        pc = ctx.pc
        gy = gy.contiguous()
        from oslo_b200.ops.gemm import matmul_nt

        gx = gw = None
        if _use_fused(gy, weight.t(), "ag"):
            from oslo_b200.ops import fused_collectives as fc

            # dX = all_gather(dY) @ W ; the gathered dY is reused for dW
            gx, gy_full = fc.ag_gemm(gy, weight.t(), pc)
        else:
            gy_full = comm.all_gather(gy, dim=0, parallel_context=pc, parallel_mode=_MODE)
            gx = matmul_nt(gy_full, weight.t()) if ctx.needs_input_grad[0] else None
        if ctx.needs_input_grad[1]:
            gw = matmul_nt(gy_full.t(), x.t())
        return gx, gw, None


def ag_linear(x, weight, parallel_context):
    """Sequence-parallel column linear on flattened tokens ``[T/tp, K] -> [T, N/tp]``."""
    return _AGLinear.apply(x, weight, parallel_context)


def linear_rs(x, weight, parallel_context):
    """Sequence-parallel row linear on flattened tokens ``[T, K/tp] -> [T/tp, N]``."""
    return _LinearRS.apply(x, weight, parallel_context)
