"""Linear layer whose weight is sharded by rows over the data-parallel group (ZeRO-3 / FSDP style), with the parameter
all-gather fused into the GEMM that consumes it.

A ZeRO-3 engine gathers a layer's parameters right before the layer runs and drops them afterwards; the gather and the
first product that reads the gathered weight are two passes over the same bytes.  Here they are one launch: with
``y = x W^T`` and ``W`` sharded by output rows, ``y^T = all_gather_rows(W_shard) x^T`` is exactly the "all-gather -> GEMM"
form of ``csrc/gemm_core.cuh`` (mode ``kModeAllGather``) with the WEIGHT as the gathered operand: every rank pushes its rows
to its peers' symmetric buffers while the tensor cores already multiply the tiles that have arrived.  The output comes
back as ``y^T`` (row-major ``[N, M]``); ``y`` is returned as its transposed view, which the GEMM kernels of this package
read as an MN-major operand without a copy.

Backward: ``dW_shard = reduce_scatter_rows(dY^T X)`` is the fused "GEMM -> reduce-scatter" kernel (the same one the
row-parallel linears use), so weight gradients never exist unsharded; ``dX = dY W`` re-gathers ``W`` (NCCL) the way ZeRO-3
does in its backward.  On CPU / gloo, or when the symmetric workspace of the group is not enabled, the same algebra runs as
collective + matmul, which is also the correctness oracle of the fused path.

This is the data-parallel counterpart of the reference's hetero ZeRO-3 parameter gathering
(oslo/torch/nn/parallel/data_parallel/zero/hetero/chunk/manager.py ``access_chunk`` all-gathers a chunk before its modules
run); the reference has no fused form.  The fused route is a switch (``FUSED_GATHER`` below) that follows the measurement.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from oslo_b200.distributed import ParallelMode


#: route the gather + product (and the weight-gradient product + reduce-scatter) through the fused kernels when the group's
#: symmetric workspace is enabled.  Off by default: on two B200s, 8192 tokens per rank, 2048 -> 8192 features, an isolated
#: forward took 0.448 ms fused against 0.282 ms for NCCL all-gather + cuBLAS (forward + backward 1.284 against 0.860 ms):
#: the weight rows are only 17 MB per rank against 275 GFLOP of product, so there is little transfer to hide, while the
#: fused kernel gives up 16 SMs to the copy role, runs the one-CTA tile and adds the row bias in a pass of its own.
#: OSLO_B200_ZERO_LINEAR_FUSED=1 (or setting this attribute) switches it on, e.g. for small per-rank batches.
FUSED_GATHER = __import__("os").environ.get("OSLO_B200_ZERO_LINEAR_FUSED", "0") == "1"


def _fused_runtime(mode):
    if not FUSED_GATHER:
        return None
    from oslo_b200.ops import fused_collectives as fc

    return fc.runtime(mode)


def _gather_rows(w_shard: torch.Tensor, group, world: int) -> torch.Tensor:
    if world == 1:
        return w_shard
    full = torch.empty((world * w_shard.shape[0],) + tuple(w_shard.shape[1:]), dtype=w_shard.dtype, device=w_shard.device)
    dist.all_gather_into_tensor(full, w_shard.contiguous(), group=group)
    return full


def _scatter_rows(full: torch.Tensor, group, world: int) -> torch.Tensor:
    if world == 1:
        return full
    out = torch.empty((full.shape[0] // world,) + tuple(full.shape[1:]), dtype=full.dtype, device=full.device)
    if full.device.type == "cpu":  # gloo has no reduce_scatter: reduce, then keep this rank's rows
        dist.all_reduce(full, group=group)
        rank = dist.get_rank(group)
        return full[rank * out.shape[0] : (rank + 1) * out.shape[0]].clone()
    dist.reduce_scatter_tensor(out, full.contiguous(), group=group)
    return out


class _ZeroLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w_shard, bias, pc, mode, average):
        group, world = pc.get_group(mode), pc.get_world_size(mode)
        x2 = x.reshape(-1, x.shape[-1])
        rt = _fused_runtime(mode) if x2.is_cuda else None
        fused = rt is not None and world > 1 and rt.ws.ag_ok(w_shard, x2)
        if fused:
            # gathered operand = the weight; "weight" operand of the kernel = the activations: y^T = W_full x^T
            y_t, _ = rt.ag_gemm(w_shard, x2, None, keep=False)
            if bias is not None:
                y_t.add_(bias.to(y_t.dtype)[:, None])
            y = y_t.t()
        else:
            w_full = _gather_rows(w_shard, group, world)
            y = torch.nn.functional.linear(x2, w_full, bias)
        ctx.save_for_backward(x2, w_shard)
        ctx.meta = (pc, mode, average, bias is not None, x.shape, fused)
        return y if x.dim() == 2 else y.unflatten(0, x.shape[:-1])

    @staticmethod
    def backward(ctx, gy):
        x2, w_shard = ctx.saved_tensors
        pc, mode, average, has_bias, x_shape, fused = ctx.meta
        group, world = pc.get_group(mode), pc.get_world_size(mode)
        g2 = gy.reshape(-1, gy.shape[-1])
        scale = 1.0 / world if average else 1.0
        gx = gw = gb = None
        if ctx.needs_input_grad[0]:
            w_full = _gather_rows(w_shard, group, world)  # re-gathered, as a ZeRO-3 backward does
            gx = torch.matmul(g2, w_full).reshape(x_shape)
        if ctx.needs_input_grad[1]:
            rt = _fused_runtime(mode) if g2.is_cuda else None
            g_t = g2.t()  # [N, M]
            if rt is not None and world > 1 and g_t.shape[0] % world == 0 and rt.ws.rs_ok(g_t, x2.t()):
                gw = rt.gemm_rs(g_t, x2.t())  # reduce_scatter_rows(dY^T X) in one kernel
            else:
                gw = _scatter_rows(torch.matmul(g_t, x2), group, world)
            if scale != 1.0:
                gw = gw * scale
        if has_bias and ctx.needs_input_grad[2]:
            gb = g2.sum(0)
            if world > 1:
                dist.all_reduce(gb, group=group)
            gb = gb * scale
        return gx, gw, gb, None, None, None


def zero_linear(x: torch.Tensor, w_shard: torch.Tensor, bias: Optional[torch.Tensor], pc, mode=ParallelMode.DATA,
                average_grads: bool = True) -> torch.Tensor:
    """``x @ all_gather_rows(w_shard)^T + bias`` over the group of ``mode``; gradients of ``w_shard`` (and ``bias``) come
    back already reduced over the group (averaged when ``average_grads``: the data-parallel convention)."""
    return _ZeroLinearFn.apply(x, w_shard, bias, pc, mode, average_grads)


class ZeroShardedLinear(nn.Module):
    """``nn.Linear`` whose weight rows are sharded over the data-parallel group; see the module docstring.

    ``from_linear`` shards an existing layer (every rank passes the same full layer); ``full_weight()`` gathers for
    checkpoints.  The bias is small and stays replicated; its gradient is all-reduced inside the backward."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, parallel_context=None, mode=ParallelMode.DATA,
                 dtype=None, device=None, average_grads: bool = True):
        super().__init__()
        self.pc, self.mode, self.average_grads = parallel_context, mode, average_grads
        world = parallel_context.get_world_size(mode)
        if out_features % world:
            raise ValueError(f"out_features {out_features} is not a multiple of the group size {world}")
        self.in_features, self.out_features, self.world = in_features, out_features, world
        self.weight = nn.Parameter(torch.empty(out_features // world, in_features, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(out_features, dtype=dtype, device=device)) if bias else None
        self.weight.oslo_zero_sharded = True  # data-parallel wrappers must not all-reduce this gradient again
        if self.bias is not None:
            self.bias.oslo_zero_sharded = True
        self.reset_parameters()

    def reset_parameters(self):
        """Same distribution as ``nn.Linear`` (bound 1 / sqrt(fan_in)); every rank draws its own rows."""
        bound = 1.0 / math.sqrt(self.in_features)
        nn.init.uniform_(self.weight, -bound, bound)
        if self.bias is not None:
            nn.init.zeros_(self.bias)

    @classmethod
    def from_linear(cls, linear: nn.Linear, parallel_context, mode=ParallelMode.DATA, average_grads: bool = True):
        m = cls(linear.in_features, linear.out_features, linear.bias is not None, parallel_context, mode,
                linear.weight.dtype, linear.weight.device, average_grads)
        rank = parallel_context.get_local_rank(mode)
        rows = linear.out_features // m.world
        with torch.no_grad():
            m.weight.copy_(linear.weight[rank * rows : (rank + 1) * rows])
            if m.bias is not None:
                m.bias.copy_(linear.bias)
        return m

    @torch.no_grad()
    def full_weight(self) -> torch.Tensor:
        return _gather_rows(self.weight.detach(), self.pc.get_group(self.mode), self.world)

    def forward(self, x):
        return zero_linear(x, self.weight, self.bias, self.pc, self.mode, self.average_grads)

    def extra_repr(self):
        return f"in_features={self.in_features}, out_features={self.out_features} (rows sharded {self.world}-way), bias={self.bias is not None}"


def shard_linears(module: nn.Module, parallel_context, mode=ParallelMode.DATA, min_features: int = 0, skip=()) -> int:
    """Replace every ``nn.Linear`` of ``module`` whose ``out_features`` divides by the group size (and is at least
    ``min_features``) by a :class:`ZeroShardedLinear` holding this rank's rows.  Returns the number replaced."""
    world = parallel_context.get_world_size(mode)
    count = 0
    for name, child in list(module.named_modules()):
        for attr, sub in list(child.named_children()):
            full = f"{name}.{attr}" if name else attr
            if type(sub) is not nn.Linear or any(full == s or full.startswith(s + ".") for s in skip):
                continue
            if sub.out_features % world or sub.out_features < min_features:
                continue
            setattr(child, attr, ZeroShardedLinear.from_linear(sub, parallel_context, mode))
            count += 1
    return count


__all__ = ["zero_linear", "ZeroShardedLinear", "shard_linears"]
