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
#: Largest tensor-parallel size at which the row-parallel side (GEMM -> reduce-scatter) uses the fused kernel.  Measured
#: back to back as isolated calls on 8 x B200 (tokens 16384, hidden 2048): the fused reduce-scatter kernels take 0.26 - 0.34 ms
#: per layer product against 0.20 - 0.28 ms for the tcgen05 GEMM followed by NCCL's in-switch reduce-scatter, while at 2 ranks
#: the fused kernel is ahead (0.32 vs 0.41 ms).  The whole 1.3B step, however, has only been measured with both sides fused
#: (47.3 ms at 8 ranks), so that stays the default; OSLO_B200_FUSED_RS_MAX_RANKS=4 moves the row-parallel side to GEMM + NCCL
#: reduce-scatter above four ranks.  The all-gather side is ahead at every size and is always fused.
FUSED_RS_MAX_RANKS = int(__import__("os").environ.get("OSLO_B200_FUSED_RS_MAX_RANKS", "8"))


def _use_fused(x, weight, kind) -> bool:
    from oslo_b200.ops import fused_collectives as fc

    if kind == "rs" and fc.runtime() is not None and fc.runtime().ws.tp > FUSED_RS_MAX_RANKS:
        return False
    return fc.available(x, weight, kind)


class _AGLinear(torch.autograd.Function):
    """y_full = all_gather(x_shard, dim 0) @ W^T.  x_shard: [T/tp, K] (tokens flattened)."""

    @staticmethod
    def forward(ctx, x, weight, pc, bias=None):
        ctx.pc = pc
        ctx.has_bias = bias is not None
        if _use_fused(x, weight, "ag"):
            from oslo_b200.ops import fused_collectives as fc

            y, x_full = fc.ag_gemm(x, weight, pc, bias=bias)  # the bias is added in the GEMM epilogue
        else:
            from oslo_b200.ops.gemm import matmul_nt

            x_full = comm.all_gather(x, dim=0, parallel_context=pc, parallel_mode=_MODE)
            y = matmul_nt(x_full, weight)
            if bias is not None:
                y = y + bias
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
        gb = None
        if ctx.has_bias and ctx.needs_input_grad[3]:
            from oslo_b200.ops.activation import colsum

            gb = colsum(gy)
        return gx, gw, None, gb


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

            # dX = all_gather(dY) @ W ; the gathered dY is reused for dW right away, so the workspace view is enough
            gx, gy_full = fc.ag_gemm(gy, weight.t(), pc, keep=False)
        else:
            gy_full = comm.all_gather(gy, dim=0, parallel_context=pc, parallel_mode=_MODE)
            gx = matmul_nt(gy_full, weight.t()) if ctx.needs_input_grad[0] else None
        if ctx.needs_input_grad[1]:
            gw = matmul_nt(gy_full.t(), x.t())
        return gx, gw, None


def ag_linear(x, weight, parallel_context, bias=None):
    """Sequence-parallel column linear on flattened tokens ``[T/tp, K] -> [T, N/tp]`` (``bias``: ``[N/tp]``, optional)."""
    return _AGLinear.apply(x, weight, parallel_context, bias)


def linear_rs(x, weight, parallel_context):
    """Sequence-parallel row linear on flattened tokens ``[T, K/tp] -> [T/tp, N]``."""
    return _LinearRS.apply(x, weight, parallel_context)


# ------------------------------------------- paired linears: two products, one collective
class _AGLinearPair(torch.autograd.Function):
    """``(y1, y2) = (X W1^T, X W2^T)`` with ``X = all_gather(x_shard)``: two column-parallel linears that read the same
    token-sharded input share ONE all-gather forward and ONE reduce-scatter backward
    (``dx = reduce_scatter(dY1 W1 + dY2 W2)``, the first product riding along as the fused kernel's addend)."""

    @staticmethod
    def forward(ctx, x, w1, w2, pc, b1=None, b2=None, gelu2=False):
        from oslo_b200.ops.gemm import gemm_bias_gelu, matmul_nt

        ctx.pc = pc
        ctx.has_b1, ctx.has_b2, ctx.gelu2 = b1 is not None, b2 is not None, gelu2
        if _use_fused(x, w1, "ag"):
            from oslo_b200.ops import fused_collectives as fc

            y1, x_full = fc.ag_gemm(x, w1, pc, bias=b1)
        else:
            x_full = comm.all_gather(x, dim=0, parallel_context=pc, parallel_mode=_MODE)
            y1 = matmul_nt(x_full, w1)
            if b1 is not None:
                y1 = y1 + b1
        pre2 = None
        if gelu2:
            y2, pre2 = gemm_bias_gelu(x_full, w2, b2)  # bias + GELU in the epilogue, pre-activation kept for backward
        else:
            y2 = matmul_nt(x_full, w2)
            if b2 is not None:
                y2 = y2 + b2
        ctx.save_for_backward(x_full, w1, w2, pre2)
        if gelu2 == "deferred":
            # the consumer of y2 applies gelu'(pre2) to the gradient it sends back (in a GEMM epilogue): hand it pre2
            ctx.mark_non_differentiable(pre2)
            return y1, y2, pre2
        return y1, y2

    @staticmethod
    def backward(ctx, g1, g2, *unused):
        from oslo_b200.ops.activation import colsum
        from oslo_b200.ops.gemm import gelu_backward, matmul_nt

        x_full, w1, w2, pre2 = ctx.saved_tensors
        pc = ctx.pc
        g1, g2 = g1.contiguous(), g2.contiguous()
        if ctx.gelu2 and ctx.gelu2 != "deferred":  # "deferred": g2 already is the gradient of the pre-activation
            g2 = gelu_backward(g2, pre2)
        gx = gw1 = gw2 = None
        if ctx.needs_input_grad[0]:
            part = matmul_nt(g1, w1.t())  # local [T, K]
            if _use_fused(g2, w2.t(), "rs"):
                from oslo_b200.ops import fused_collectives as fc

                gx = fc.gemm_rs(g2, w2.t(), pc, addend=part)
            else:
                part = part + matmul_nt(g2, w2.t())
                gx = comm.reduce_scatter(part, dim=0, parallel_context=pc, parallel_mode=_MODE)
        if ctx.needs_input_grad[1]:
            gw1 = matmul_nt(g1.t(), x_full.t())
        if ctx.needs_input_grad[2]:
            gw2 = matmul_nt(g2.t(), x_full.t())
        gb1 = colsum(g1) if (ctx.has_b1 and ctx.needs_input_grad[4]) else None
        gb2 = colsum(g2) if (ctx.has_b2 and ctx.needs_input_grad[5]) else None
        return gx, gw1, gw2, None, gb1, gb2, None


class _LinearPairRS(torch.autograd.Function):
    """``y_shard = reduce_scatter(X1 W1^T + X2 W2^T)``: two row-parallel linears whose outputs are summed right after
    (attention output and MLP output of a parallel-residual block) share ONE reduce-scatter forward and ONE all-gather
    of ``dY`` backward."""

    @staticmethod
    def forward(ctx, x1, w1, x2, w2, pc, x2_pre=None):
        from oslo_b200.ops.gemm import matmul_nt

        ctx.pc = pc
        ctx.has_pre = x2_pre is not None
        ctx.save_for_backward(x1, w1, x2, w2, *([x2_pre] if x2_pre is not None else []))
        if _use_fused(x2, w2, "rs"):
            from oslo_b200.ops import fused_collectives as fc

            # the second product rides along: as a ready [T, N] addend in the one-kernel transports, block by block
            # (accumulated into the same staging block) with the copy-engine transport
            return fc.gemm_rs(x2, w2, pc, pair=(x1, w1))
        part = matmul_nt(x1, w1) + matmul_nt(x2, w2)
        return comm.reduce_scatter(part, dim=0, parallel_context=pc, parallel_mode=_MODE)

    @staticmethod
    def backward(ctx, gy):
        from oslo_b200.ops.gemm import matmul_nt

        x1, w1, x2, w2 = ctx.saved_tensors[:4]
        pre = ctx.saved_tensors[4] if ctx.has_pre else None  # x2 = gelu(pre): the gradient returned for x2 is d(pre)
        pc = ctx.pc
        gy = gy.contiguous()
        if _use_fused(gy, w2.t(), "ag"):
            from oslo_b200.ops import fused_collectives as fc

            # consumed by the GEMMs below before two more fused calls; gelu'(pre) rides in this GEMM's epilogue
            gx2, gy_full = fc.ag_gemm(gy, w2.t(), pc, keep=False, gelu_grad_of=pre)
        else:
            gy_full = comm.all_gather(gy, dim=0, parallel_context=pc, parallel_mode=_MODE)
            gx2 = matmul_nt(gy_full, w2.t())
            if pre is not None:
                from oslo_b200.ops.gemm import gelu_backward

                gx2 = gelu_backward(gx2, pre)
        gx1 = matmul_nt(gy_full, w1.t()) if ctx.needs_input_grad[0] else None
        gw1 = matmul_nt(gy_full.t(), x1.t()) if ctx.needs_input_grad[1] else None
        gw2 = matmul_nt(gy_full.t(), x2.t()) if ctx.needs_input_grad[3] else None
        return gx1, gw1, gx2, gw2, None, None


def ag_linear_pair(x, w1, w2, parallel_context, b1=None, b2=None, gelu2=False):
    """Two sequence-parallel column linears on the same input: ``[T/tp, K] -> ([T, N1/tp] (+ b1), [T, N2/tp] (+ b2))``;
    ``gelu2`` applies the tanh GELU to the second output inside its GEMM epilogue.  ``gelu2="deferred"`` additionally
    returns the pre-activation as a third output and expects the gradient that comes back for the second output to be the
    gradient of that PRE-activation: pass it to :func:`linear_pair_rs` as ``x2_pre``, whose backward applies ``gelu'`` in
    the epilogue of its gradient GEMM."""
    return _AGLinearPair.apply(x, w1, w2, parallel_context, b1, b2, gelu2)


def linear_pair_rs(x1, w1, x2, w2, parallel_context, x2_pre=None):
    """Two sequence-parallel row linears summed: ``([T, K1/tp], [T, K2/tp]) -> [T/tp, N]``.  With ``x2_pre`` (``x2`` is
    ``gelu_tanh(x2_pre)``, produced by ``ag_linear_pair(..., gelu2="deferred")``) the gradient returned for ``x2`` is the
    gradient of ``x2_pre``."""
    return _LinearPairRS.apply(x1, w1, x2, w2, parallel_context, x2_pre)
