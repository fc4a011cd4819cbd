"""Collective wrappers with ``dim`` semantics on top of ``torch.distributed``.

All functions take ``parallel_context`` and ``parallel_mode`` and resolve the
communicator there; ``on_cpu=True`` uses the gloo twin of the group;
``async_op=True`` returns ``(tensor, work)``.  Groups of size 1 short-circuit.

The single-buffer collectives (``all_gather_into_tensor`` /
``reduce_scatter_tensor``) are used whenever the backend offers them so a gather
along ``dim != 0`` costs one permute instead of ``world`` chunk copies.

Parity: ``oslo/torch/distributed/nn/functional.py:43-283``.
"""
from __future__ import annotations

from typing import Any, List, Optional

import torch
import torch.distributed as dist
from torch import Tensor

from .parallel_mode import ParallelMode

ReduceOp = dist.ReduceOp


def _group(pc, mode, on_cpu=False):
    return pc.get_cpu_group(mode) if on_cpu else pc.get_group(mode)


def _ret(out, work, async_op):
    return (out, work) if async_op else out


def all_gather(
    tensor: Tensor,
    dim: int = -1,
    on_cpu: bool = False,
    async_op: bool = False,
    parallel_context=None,
    parallel_mode: ParallelMode = ParallelMode.GLOBAL,
):
    """Concatenate every rank's ``tensor`` along ``dim``."""
    world = parallel_context.get_world_size(parallel_mode)
    if world == 1:
        return _ret(tensor, None, async_op)
    group = _group(parallel_context, parallel_mode, on_cpu)
    dim = dim % tensor.dim()
    src = tensor.contiguous()
    flat = torch.empty((world,) + tuple(src.shape), dtype=src.dtype, device=src.device)
    # a gather along dim != 0 needs a permute after the data has landed, so only
    # dim == 0 can be left in flight; other dims complete before returning.
    in_flight = async_op and dim == 0
    work = dist.all_gather_into_tensor(flat.view(-1), src.view(-1), group=group, async_op=in_flight)
    if dim == 0:
        out = flat.view((world * src.shape[0],) + tuple(src.shape[1:]))
        return _ret(out, work, async_op)
    shape = list(src.shape)
    shape[dim] *= world
    out = flat.movedim(0, dim).reshape(shape)  # [..., world, d, ...] -> [..., world*d, ...]
    return _ret(out, _DoneWork(), async_op)


class _DoneWork:
    """Stand-in handle for an operation that completed before returning."""

    def wait(self):
        return True

    def is_completed(self):
        return True


def reduce_scatter(
    tensor: Tensor,
    dim: int = -1,
    op=ReduceOp.SUM,
    on_cpu: bool = False,
    async_op: bool = False,
    parallel_context=None,
    parallel_mode: ParallelMode = ParallelMode.GLOBAL,
):
    """Sum over ranks, keep this rank's chunk along ``dim``."""
    world = parallel_context.get_world_size(parallel_mode)
    if world == 1:
        return _ret(tensor, None, async_op)
    group = _group(parallel_context, parallel_mode, on_cpu)
    dim = dim % tensor.dim()
    if tensor.shape[dim] % world:
        raise ValueError(f"reduce_scatter: dim {dim} of size {tensor.shape[dim]} not divisible by {world}")
    if dim == 0:
        src = tensor.contiguous()
    else:
        shape = list(tensor.shape)
        shape[dim : dim + 1] = [world, shape[dim] // world]
        src = tensor.reshape(shape).movedim(dim, 0).contiguous()
    out_shape = list(tensor.shape)
    out_shape[dim] //= world
    out = torch.empty(out_shape, dtype=tensor.dtype, device=tensor.device)
    if dist.get_backend(group) == "gloo":
        # gloo lacks reduce_scatter: all-reduce then slice (CPU correctness path only)
        buf = src.clone()
        dist.all_reduce(buf, op=op, group=group)
        rank = parallel_context.get_local_rank(parallel_mode)
        n = out.numel()
        out.view(-1).copy_(buf.view(-1)[rank * n : (rank + 1) * n])
        return _ret(out, _DoneWork(), async_op)
    work = dist.reduce_scatter_tensor(out.view(-1), src.view(-1), op=op, group=group, async_op=async_op)
    return _ret(out, work, async_op)


def all_reduce(
    tensor: Tensor,
    op=ReduceOp.SUM,
    on_cpu: bool = False,
    async_op: bool = False,
    parallel_context=None,
    parallel_mode: ParallelMode = ParallelMode.GLOBAL,
):
    world = parallel_context.get_world_size(parallel_mode)
    if world == 1:
        return _ret(tensor, None, async_op)
    group = _group(parallel_context, parallel_mode, on_cpu)
    if not tensor.is_contiguous():
        tensor = tensor.contiguous()
    work = dist.all_reduce(tensor, op=op, group=group, async_op=async_op)
    return _ret(tensor, work, async_op)


def broadcast(
    tensor: Tensor,
    src: int,
    on_cpu: bool = False,
    async_op: bool = False,
    parallel_context=None,
    parallel_mode: ParallelMode = ParallelMode.GLOBAL,
):
    """``src`` is a global rank."""
    world = parallel_context.get_world_size(parallel_mode)
    if world == 1:
        return _ret(tensor, None, async_op)
    group = _group(parallel_context, parallel_mode, on_cpu)
    if not tensor.is_contiguous():
        tensor = tensor.contiguous()
    work = dist.broadcast(tensor, src=src, group=group, async_op=async_op)
    return _ret(tensor, work, async_op)


def reduce(
    tensor: Tensor,
    dst: int,
    op=ReduceOp.SUM,
    on_cpu: bool = False,
    async_op: bool = False,
    parallel_context=None,
    parallel_mode: ParallelMode = ParallelMode.GLOBAL,
):
    """``dst`` is a global rank."""
    world = parallel_context.get_world_size(parallel_mode)
    if world == 1:
        return _ret(tensor, None, async_op)
    group = _group(parallel_context, parallel_mode, on_cpu)
    if not tensor.is_contiguous():
        tensor = tensor.contiguous()
    work = dist.reduce(tensor, dst=dst, op=op, group=group, async_op=async_op)
    return _ret(tensor, work, async_op)


def scatter(
    tensor: Tensor,
    dim: int = -1,
    parallel_context=None,
    parallel_mode: ParallelMode = ParallelMode.GLOBAL,
) -> Tensor:
    """Keep this rank's chunk along ``dim`` (no communication)."""
    world = parallel_context.get_world_size(parallel_mode)
    if world == 1:
        return tensor
    rank = parallel_context.get_local_rank(parallel_mode)
    if tensor.shape[dim] % world:
        raise ValueError(f"scatter: dim {dim} of size {tensor.shape[dim]} not divisible by {world}")
    return tensor.chunk(world, dim=dim)[rank].contiguous()


def all_to_all(
    tensor: Tensor,
    output_split_sizes: Optional[List[int]] = None,
    input_split_sizes: Optional[List[int]] = None,
    on_cpu: bool = False,
    parallel_context=None,
    parallel_mode: ParallelMode = ParallelMode.GLOBAL,
) -> Tensor:
    """All-to-all along dim 0.  gloo has no all_to_all: emulated with one all-gather."""
    world = parallel_context.get_world_size(parallel_mode)
    if world == 1:
        return tensor
    group = _group(parallel_context, parallel_mode, on_cpu)
    tensor = tensor.contiguous()
    if dist.get_backend(group) != "gloo":
        if output_split_sizes is None:
            out = torch.empty_like(tensor)
        else:
            out = tensor.new_empty((sum(output_split_sizes),) + tuple(tensor.shape[1:]))
        dist.all_to_all_single(out, tensor, output_split_sizes, input_split_sizes, group=group)
        return out
    rank = parallel_context.get_local_rank(parallel_mode)
    if input_split_sizes is None:
        gathered = [torch.empty_like(tensor) for _ in range(world)]
        dist.all_gather(gathered, tensor, group=group)
        return torch.cat([g.chunk(world, dim=0)[rank] for g in gathered], dim=0)
    splits = [None] * world
    dist.all_gather_object(splits, list(input_split_sizes), group=group)
    rows = [sum(s) for s in splits]
    pieces = []
    for r in range(world):
        buf = tensor.new_empty((rows[r],) + tuple(tensor.shape[1:])) if r != rank else tensor
        dist.broadcast(buf, src=parallel_context.get_ranks_in_group(parallel_mode)[r], group=group)
        start = sum(splits[r][:rank])
        pieces.append(buf[start : start + splits[r][rank]])
    return torch.cat(pieces, dim=0)


def scatter_object_list(
    scatter_object_output_list: List[Any],
    scatter_object_input_list: Optional[List[Any]],
    src: int = 0,
    parallel_context=None,
    parallel_mode: ParallelMode = ParallelMode.GLOBAL,
):
    """Scatter picklable objects from global rank ``src`` (uses the gloo twin under NCCL)."""
    world = parallel_context.get_world_size(parallel_mode)
    if world == 1:
        scatter_object_output_list[0] = scatter_object_input_list[0]
        return
    group = parallel_context.get_cpu_group(parallel_mode)
    dist.scatter_object_list(scatter_object_output_list, scatter_object_input_list, src=src, group=group)


def barrier(parallel_context=None, parallel_mode: ParallelMode = ParallelMode.GLOBAL, on_cpu: bool = False):
    if parallel_context.get_world_size(parallel_mode) > 1:
        dist.barrier(group=_group(parallel_context, parallel_mode, on_cpu))


def send(data: Any, src_rank: int, dst_rank: int, parallel_context=None, parallel_mode=ParallelMode.GLOBAL):
    from .p2p import P2P

    return P2P().send(data, src_rank, dst_rank, parallel_context, parallel_mode)


def recv(src_rank: int, dst_rank: int, parallel_context=None, parallel_mode=ParallelMode.GLOBAL):
    from .p2p import P2P

    return P2P().recv(src_rank, dst_rank, parallel_context, parallel_mode)


def ring_qk(sub_q: Tensor, sub_k: Tensor, parallel_context):
    from .ring_attention import RingQK

    return RingQK.apply(sub_q, sub_k, parallel_context)


def ring_av(sub_attn: Tensor, sub_v: Tensor, parallel_context):
    from .ring_attention import RingAV

    return RingAV.apply(sub_attn, sub_v, parallel_context)
