"""Chunks: fixed-size flat buffers of parameters, each sharded evenly over the data-parallel group (ZeRO-3).

A chunk is either *scattered* (every rank holds ``1/dp`` of it, possibly in pinned host memory) or *gathered* (the
full buffer is materialised on the compute device and the parameters are views into it).  ``ChunkManager`` packs
parameters in registration order, chooses the chunk size that wastes the least padding, and implements
``access`` (all-gather), ``release`` and ``reduce`` (reduce-scatter of gradients).

Parity: oslo/torch/nn/parallel/data_parallel/zero/hetero/chunk/{chunk,manager,utils}.py.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch
import torch.distributed as dist


class Chunk:
    def __init__(self, size: int, dtype, world: int, rank: int, group, compute_device, shard_device, keep_gathered=False):
        assert size % world == 0
        self.size, self.dtype = size, dtype
        self.world, self.rank, self.group = world, rank, group
        self.compute_device, self.shard_device = compute_device, shard_device
        self.keep_gathered = keep_gathered
        self.params: List[torch.nn.Parameter] = []
        self.offsets: List[int] = []
        self.used = 0
        self.full: Optional[torch.Tensor] = torch.zeros(size, dtype=dtype, device=compute_device)
        self.shard: Optional[torch.Tensor] = None
        self.grad_shard: Optional[torch.Tensor] = None
        self.full_grad: Optional[torch.Tensor] = None
        self.pending_grads = 0

    @property
    def shard_size(self):
        return self.size // self.world

    def can_fit(self, numel: int) -> bool:
        return self.used + numel <= self.size

    def append(self, p: torch.nn.Parameter):
        n = p.numel()
        self.full[self.used : self.used + n].copy_(p.data.reshape(-1).to(self.full.device))
        self.params.append(p)
        self.offsets.append(self.used)
        self.used += n

    def close(self):
        """Finish packing: keep only this rank's shard."""
        lo = self.rank * self.shard_size
        shard = self.full[lo : lo + self.shard_size].clone().to(self.shard_device)
        if self.shard_device.type == "cpu" and torch.cuda.is_available():
            shard = shard.pin_memory()
        self.shard = shard
        self._point_params(self.full)
        if not self.keep_gathered:
            self.release()

    def _point_params(self, buf: Optional[torch.Tensor]):
        for p, off in zip(self.params, self.offsets):
            if buf is None:
                p.data = torch.empty(0, dtype=p.dtype, device=self.compute_device)
            else:
                p.data = buf[off : off + p.oslo_numel].view(p.oslo_shape)

    @property
    def is_gathered(self):
        return self.full is not None

    def access(self):
        """All-gather the shards into a full buffer on the compute device."""
        if self.full is not None:
            return
        local = self.shard.to(self.compute_device, non_blocking=True)
        full = torch.empty(self.size, dtype=self.dtype, device=self.compute_device)
        if self.world > 1:
            dist.all_gather_into_tensor(full, local.contiguous(), group=self.group)
        else:
            full.copy_(local)
        self.full = full
        self._point_params(full)

    def release(self):
        if self.keep_gathered or self.full is None:
            return
        self.full = None
        self._point_params(None)

    def write_back(self):
        """After an optimizer step on the shard, refresh a gathered copy if one is held."""
        if self.full is not None:
            if self.world > 1:
                dist.all_gather_into_tensor(self.full, self.shard.to(self.compute_device).contiguous(), group=self.group)
            else:
                self.full.copy_(self.shard.to(self.compute_device))

    def reduce_grads(self):
        """Average the gradients over the group and keep this rank's slice (reduce-scatter)."""
        g = torch.zeros(self.size, dtype=self.dtype, device=self.compute_device)
        for p, off in zip(self.params, self.offsets):
            if p.grad is not None:
                g[off : off + p.oslo_numel].copy_(p.grad.reshape(-1))
                p.grad = None
        g.div_(self.world)
        if self.world > 1:
            if dist.get_backend(self.group) == "gloo":
                dist.all_reduce(g, group=self.group)
                out = g[self.rank * self.shard_size : (self.rank + 1) * self.shard_size].clone()
            else:
                out = torch.empty(self.shard_size, dtype=self.dtype, device=self.compute_device)
                dist.reduce_scatter_tensor(out, g, group=self.group)
        else:
            out = g
        out = out.to(self.shard_device)
        self.grad_shard = out if self.grad_shard is None else self.grad_shard + out


def search_chunk_size(numels: Sequence[int], world: int, min_mb: float = 1.0, max_mb: float = 64.0, elem_bytes: int = 2,
                      step: int = 1024) -> int:
    """Chunk size (elements, multiple of ``world * step``) minimising padding waste for this parameter list."""
    unit = world * step
    lo = max(unit, int(min_mb * 2**20 / elem_bytes) // unit * unit)
    hi = max(lo, int(max_mb * 2**20 / elem_bytes) // unit * unit)
    biggest = max(numels) if numels else unit
    lo = max(lo, (biggest + unit - 1) // unit * unit)
    hi = max(hi, lo)
    best, best_waste = lo, None
    size = lo
    while size <= hi:
        used, waste = 0, 0
        for n in numels:
            if used + n > size:
                waste += size - used
                used = 0
            used += n
        waste += size - used
        if best_waste is None or waste < best_waste:
            best, best_waste = size, waste
        size += max(unit, (hi - lo) // 64 // unit * unit)
    return best


class ChunkManager:
    def __init__(self, world: int, rank: int, group, compute_device, shard_device, chunk_size: int):
        self.world, self.rank, self.group = world, rank, group
        self.compute_device, self.shard_device, self.chunk_size = compute_device, shard_device, chunk_size
        self.chunks: List[Chunk] = []
        self.param_to_chunk: Dict[int, Chunk] = {}
        self.gather_calls = 0
        self.before_access = None  # optional hook(chunk): the memory manager adjusts the layout before a gather

    def register(self, params: Sequence[torch.nn.Parameter], keep_gathered_small: bool = False):
        cur: Optional[Chunk] = None
        for p in params:
            p.oslo_shape, p.oslo_numel = p.shape, p.numel()
            if cur is None or cur.dtype != p.dtype or not cur.can_fit(p.numel()):
                if cur is not None:
                    cur.close()
                cur = Chunk(self.chunk_size, p.dtype, self.world, self.rank, self.group, self.compute_device, self.shard_device)
                self.chunks.append(cur)
            cur.append(p)
            self.param_to_chunk[id(p)] = cur
        if cur is not None:
            cur.close()

    def chunks_of(self, params) -> List[Chunk]:
        seen, out = set(), []
        for p in params:
            c = self.param_to_chunk.get(id(p))
            if c is not None and id(c) not in seen:
                seen.add(id(c))
                out.append(c)
        return out

    def access(self, chunks):
        for c in chunks:
            if not c.is_gathered:
                if self.before_access is not None:
                    self.before_access(c)
                self.gather_calls += 1
                c.access()

    def release(self, chunks):
        for c in chunks:
            c.release()

    def total_shard_bytes(self):
        return sum(c.shard.numel() * c.shard.element_size() for c in self.chunks)
