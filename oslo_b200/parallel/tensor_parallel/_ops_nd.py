"""Autograd-aware collectives shared by the 2D / 2.5D / 3D tensor-parallel layers.

Every primitive pairs a forward collective with its adjoint in backward (all-gather <-> reduce-scatter,
all-reduce <-> identity, ...), so the N-D linears are written as plain compositions of these primitives and
``ops.gemm.linear``; autograd then derives exactly the backward communication the reference hand-codes in its
``Matmul_*`` functions (oslo/torch/nn/parallel/tensor_parallel/_2d/_ops.py:222-702, _3d/_ops.py:35-402).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from oslo_b200.distributed import ParallelMode, comm


class _AllGather(torch.autograd.Function):
    """all-gather along ``dim`` forward, reduce-scatter backward."""

    @staticmethod
    def forward(ctx, x, dim, mode, pc):
        ctx.dim, ctx.mode, ctx.pc = dim, mode, pc
        return comm.all_gather(x, dim=dim, parallel_context=pc, parallel_mode=mode)

    @staticmethod
    def backward(ctx, g):
        return comm.reduce_scatter(g.contiguous(), dim=ctx.dim, parallel_context=ctx.pc, parallel_mode=ctx.mode), None, None, None


class _ReduceScatter(torch.autograd.Function):
    """reduce-scatter along ``dim`` forward, all-gather backward."""

    @staticmethod
    def forward(ctx, x, dim, mode, pc):
        ctx.dim, ctx.mode, ctx.pc = dim, mode, pc
        return comm.reduce_scatter(x.contiguous(), dim=dim, parallel_context=pc, parallel_mode=mode)

    @staticmethod
    def backward(ctx, g):
        return comm.all_gather(g.contiguous(), dim=ctx.dim, parallel_context=ctx.pc, parallel_mode=ctx.mode), None, None, None


class _GatherReplicated(torch.autograd.Function):
    """all-gather forward; backward keeps this rank's slice (the consumers of the result are replicated)."""

    @staticmethod
    def forward(ctx, x, dim, mode, pc):
        ctx.dim, ctx.mode, ctx.pc = dim, mode, pc
        return comm.all_gather(x, dim=dim, parallel_context=pc, parallel_mode=mode)

    @staticmethod
    def backward(ctx, g):
        return comm.scatter(g, dim=ctx.dim, parallel_context=ctx.pc, parallel_mode=ctx.mode), None, None, None


class _AllReduce(torch.autograd.Function):
    """sum over the group forward, identity backward."""

    @staticmethod
    def forward(ctx, x, mode, pc):
        return comm.all_reduce(x.clone(), parallel_context=pc, parallel_mode=mode)

    @staticmethod
    def backward(ctx, g):
        return g, None, None


class _Copy(torch.autograd.Function):
    """identity forward, sum over the group backward (a replicated tensor feeding rank-specific work)."""

    @staticmethod
    def forward(ctx, x, mode, pc):
        ctx.mode, ctx.pc = mode, pc
        return x

    @staticmethod
    def backward(ctx, g):
        return comm.all_reduce(g.contiguous().clone(), parallel_context=ctx.pc, parallel_mode=ctx.mode), None, None


def all_gather(x, dim, mode, pc):
    if pc.get_world_size(mode) == 1:
        return x
    return _AllGather.apply(x, dim, mode, pc)


def reduce_scatter(x, dim, mode, pc):
    if pc.get_world_size(mode) == 1:
        return x
    return _ReduceScatter.apply(x, dim, mode, pc)


def gather_replicated(x, dim, mode, pc):
    if pc.get_world_size(mode) == 1:
        return x
    return _GatherReplicated.apply(x, dim, mode, pc)


def all_reduce(x, mode, pc):
    if pc.get_world_size(mode) == 1:
        return x
    return _AllReduce.apply(x, mode, pc)


def copy_to_group(x, mode, pc):
    if pc.get_world_size(mode) == 1:
        return x
    return _Copy.apply(x, mode, pc)


def gather_ids(ids, dim, mode, pc):
    """All-gather integer inputs (no gradient)."""
    if pc.get_world_size(mode) == 1:
        return ids
    return comm.all_gather(ids, dim=dim, parallel_context=pc, parallel_mode=mode)


# ------------------------------------------------------------------ sharded normalisation
class _ShardedNormStats(torch.autograd.Function):
    """Row sums of x (and x^2) over a hidden dim that is sharded over ``mode``: one all-reduce of both."""

    @staticmethod
    def forward(ctx, x, mode, pc, rms):
        xf = x.float()
        s2 = (xf * xf).sum(-1, keepdim=True)
        if rms:
            stats = s2
        else:
            stats = torch.cat([xf.sum(-1, keepdim=True), s2], dim=-1)
        stats = comm.all_reduce(stats.contiguous(), parallel_context=pc, parallel_mode=mode)
        ctx.save_for_backward(x)
        ctx.rms, ctx.mode, ctx.pc = rms, mode, pc
        return stats

    @staticmethod
    def backward(ctx, g):
        # each rank's g is the sensitivity of ITS hidden shard to the shared statistics: sum them (the adjoint of
        # an all-reduce whose result every rank consumes), then d(sum x)/dx = 1 and d(sum x^2)/dx = 2x
        (x,) = ctx.saved_tensors
        g = comm.all_reduce(g.contiguous().clone(), parallel_context=ctx.pc, parallel_mode=ctx.mode)
        xf = x.float()
        if ctx.rms:
            gx = 2.0 * xf * g
        else:
            gx = g[..., 0:1] + 2.0 * xf * g[..., 1:2]
        return gx.to(x.dtype), None, None, None


def sharded_norm(x, weight, bias, full_dim: int, eps: float, rms: bool, pc, mode):
    """LayerNorm / RMSNorm over a hidden dimension of global size ``full_dim`` sharded over ``mode``."""
    if pc.get_world_size(mode) == 1:
        from oslo_b200.ops.norm import layer_norm, rms_norm

        return rms_norm(x, x.shape[-1], weight, eps) if rms else layer_norm(x, x.shape[-1], weight, bias, eps)
    stats = _ShardedNormStats.apply(x, mode, pc, rms)
    xf = x.float()
    if rms:
        var = stats / full_dim
        y = xf * torch.rsqrt(var + eps)
    else:
        mean = stats[..., 0:1] / full_dim
        var = stats[..., 1:2] / full_dim - mean * mean
        y = (xf - mean) * torch.rsqrt(var.clamp_min(0) + eps)
    if weight is not None:
        y = y * weight.float()
    if bias is not None:
        y = y + bias.float()
    return y.to(x.dtype)
