"""Shard / merge arithmetic for tensor-parallel parameters.

Every sharded parameter carries a :class:`ShardSpec`: the ordered list of (mode, dim, parts) splits applied
to the full tensor, plus the unpadded full shape.  ``merge`` inverts the splits with all-gathers, which is
all ``deparallelize`` (checkpoint merging) needs — no per-layer-type code.

Layout facts reproduced for checkpoint compatibility with the reference:
* fused QKV weights are split per part (``[q|k|v]`` each sliced), not as one block
  (oslo/torch/nn/parallel/tensor_parallel/_1d/_wrapper.py:141-147);
* 2D ``W.chunk(q, dim=1)[row].chunk(q, dim=0)[col]`` (…/_2d/_wrapper.py:235-281);
* 3D ``W.chunk(c, 1)[out].chunk(c, 0)[in].chunk(c, 0)[wt]`` (…/_3d/_wrapper.py:252-300).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Tuple

import torch

from oslo_b200.distributed import ParallelMode, comm


@dataclass
class Split:
    mode: ParallelMode
    dim: int
    parts: int = 1  # >1: the dim is ``parts`` concatenated blocks, each split separately (fused QKV)


@dataclass
class ShardSpec:
    splits: List[Split] = field(default_factory=list)
    full_shape: Optional[Tuple[int, ...]] = None  # unpadded shape of the merged tensor


def split_tensor(t: torch.Tensor, dim: int, world: int, rank: int, parts: int = 1) -> torch.Tensor:
    if world == 1:
        return t
    if parts == 1:
        if t.shape[dim] % world:
            raise ValueError(f"dim {dim} of size {t.shape[dim]} is not divisible by {world}")
        return t.chunk(world, dim=dim)[rank].contiguous()
    blocks = t.chunk(parts, dim=dim)
    return torch.cat([b.chunk(world, dim=dim)[rank] for b in blocks], dim=dim).contiguous()


def shard(t: torch.Tensor, spec: ShardSpec, pc) -> torch.Tensor:
    for s in spec.splits:
        t = split_tensor(t, s.dim, pc.get_world_size(s.mode), pc.get_local_rank(s.mode), s.parts)
    return t


def merge(t: torch.Tensor, spec: ShardSpec, pc) -> torch.Tensor:
    """All-gather the shards back into the full tensor (inverse of :func:`shard`), cropping padding."""
    for s in reversed(spec.splits):
        world = pc.get_world_size(s.mode)
        if world == 1:
            continue
        g = comm.all_gather(t.contiguous(), dim=s.dim, parallel_context=pc, parallel_mode=s.mode)
        if s.parts > 1:
            # gathered layout: [rank0: p0 p1 p2 | rank1: p0 p1 p2 ...] -> [p0: r0 r1 .. | p1: ...]
            per_rank = g.chunk(world, dim=s.dim)
            pieces = [r.chunk(s.parts, dim=s.dim) for r in per_rank]
            g = torch.cat([pieces[r][p] for p in range(s.parts) for r in range(world)], dim=s.dim)
        t = g
    if spec.full_shape is not None and tuple(t.shape) != tuple(spec.full_shape):
        t = t[tuple(slice(0, n) for n in spec.full_shape)].contiguous()
    return t


def pad_dim(t: torch.Tensor, dim: int, multiple: int) -> torch.Tensor:
    n = t.shape[dim]
    target = (n + multiple - 1) // multiple * multiple
    if target == n:
        return t
    shape = list(t.shape)
    shape[dim] = target - n
    return torch.cat([t, t.new_zeros(shape)], dim=dim)
