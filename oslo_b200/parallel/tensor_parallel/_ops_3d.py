"""3-D tensor-parallel ops on a ``c x c x c`` cube; rank ``(i, j, k)`` = ranks in (WEIGHT, INPUT, OUTPUT) groups.

Layouts (as the reference): activations ``[b/c^2 (i, j), s, h/c (k)]``; ``Linear3D`` weight
``[out/c^2 (j, i), in/c (k)]``, bias ``[out/c (j)]``.

    X_i  = all_gather(x over INPUT, batch)       [b/c (i), s, in/c (k)]
    W_j  = all_gather(W over WEIGHT, out)        [out/c (j), in/c (k)]
    P    = X_i W_j^T                             partial over k
    Y    = reduce_scatter(P over OUTPUT, batch)  [b/c^2 (i, k), s, out/c (j)]  (+ bias_j)
    out  = swap(j <-> k)                         [b/c^2 (i, j), s, out/c (k)]

The last step is a pairwise exchange with rank ``(i, k, j)``; the reference pays a c^3-way all-gather for the
same permutation (``transpose_3d``, oslo/.../_3d/_ops.py:18-32).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from oslo_b200.distributed import ParallelMode
from oslo_b200.ops.gemm import linear

from . import _ops_nd as nd

INPUT, WEIGHT, OUTPUT = ParallelMode.TENSOR_3D_INPUT, ParallelMode.TENSOR_3D_WEIGHT, ParallelMode.TENSOR_3D_OUTPUT


def _swap_partner(pc) -> int:
    """Global rank of ``(i, k, j)`` for this rank ``(i, j, k)``."""
    c = pc.cubic_dim
    i = pc.get_local_rank(WEIGHT)
    j = pc.get_local_rank(INPUT)
    k = pc.get_local_rank(OUTPUT)
    base = pc.get_ranks_in_group(ParallelMode.TENSOR_3D)[0]
    return base + i + c * (k + c * j)


def _exchange(t, pc):
    partner = _swap_partner(pc)
    me = pc.get_global_rank()
    if partner == me:
        return t
    t = t.contiguous()
    out = torch.empty_like(t)
    group = pc.get_group(ParallelMode.TENSOR_3D)
    ops = [dist.P2POp(dist.isend, t, partner, group), dist.P2POp(dist.irecv, out, partner, group)]
    if me > partner:
        ops.reverse()
    for w in dist.batch_isend_irecv(ops):
        w.wait()
    return out


class _Swap3D(torch.autograd.Function):
    """Exchange tensors between ranks (i, j, k) and (i, k, j); self-adjoint."""

    @staticmethod
    def forward(ctx, t, pc):
        ctx.pc = pc
        return _exchange(t, pc)

    @staticmethod
    def backward(ctx, g):
        return _exchange(g, ctx.pc), None


def transpose_3d(t, pc):
    if pc.cubic_dim == 1:
        return t
    return _Swap3D.apply(t, pc)


class _GatherLinearScatter3D(torch.autograd.Function):
    """``reduce_scatter_OUTPUT(all_gather_INPUT(x) W^T)`` as ONE kernel (``oslo_ag_gemm_rs``): copy CTAs pull the other
    INPUT ranks' token blocks while the GEMM CTAs multiply, and each finished tile is TMA-stored straight into the OUTPUT
    rank that owns its rows.  Backward: all-gather(dY over OUTPUT), two GEMMs, reduce-scatter(dX over INPUT)."""

    @staticmethod
    def forward(ctx, x, wg, pc):
        from oslo_b200.ops import fused_collectives as fc

        ctx.pc, ctx.shape = pc, x.shape
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        y, x_full = fc.ag_gemm_rs(x2, wg, INPUT, OUTPUT)
        ctx.save_for_backward(x_full, wg)
        return y.view(*x.shape[:-1], y.shape[-1])

    @staticmethod
    def backward(ctx, g):
        from oslo_b200.distributed import comm
        from oslo_b200.ops.gemm import matmul_nt

        x_full, wg = ctx.saved_tensors
        pc = ctx.pc
        g2 = g.reshape(-1, g.shape[-1]).contiguous()
        g_full = comm.all_gather(g2, dim=0, parallel_context=pc, parallel_mode=OUTPUT)
        gx = gw = None
        if ctx.needs_input_grad[0]:
            gx_full = matmul_nt(g_full, wg.t())
            gx = comm.reduce_scatter(gx_full, dim=0, parallel_context=pc, parallel_mode=INPUT).view(ctx.shape)
        if ctx.needs_input_grad[1]:
            gw = matmul_nt(g_full.t(), x_full.t())
        return gx, gw, None


def linear_3d(x, weight, bias, pc):
    wg = nd.all_gather(weight, 0, WEIGHT, pc)
    fused = False
    if x.is_cuda and pc.cubic_dim > 1:
        from oslo_b200.ops import fused_collectives as fc

        fused = fc.gather_scatter_available(x.reshape(-1, x.shape[-1]), wg, INPUT, OUTPUT)
    if fused:
        y = _GatherLinearScatter3D.apply(x, wg, pc)
    else:
        xg = nd.all_gather(x, 0, INPUT, pc)
        partial = linear(xg, wg)
        y = nd.reduce_scatter(partial, 0, OUTPUT, pc)
    if bias is not None:
        y = y + bias
    return transpose_3d(y, pc)


def gather_output_3d(t, pc):
    """Full ``[b, s, out]`` on every rank."""
    t = nd.gather_replicated(t, -1, OUTPUT, pc)
    t = nd.gather_replicated(t, 0, INPUT, pc)
    return nd.gather_replicated(t, 0, WEIGHT, pc)


def gather_batch_3d(ids, mode, pc):
    return nd.gather_ids(ids, 0, mode, pc)


def all_gather_weight_3d(w, dim, mode, pc):
    return nd.all_gather(w, dim, mode, pc)


def reduce_scatter_tensor_3d(t, dim, mode, pc):
    return nd.reduce_scatter(t, dim, mode, pc)


def replicated_weight_3d(w, pc):
    """A weight replicated over (WEIGHT, INPUT) used on rank-specific batches; its gradient is synchronised by
    the wrapper's replicated-gradient pass, so forward is the identity."""
    return w
