"""Chunk-based ZeRO-3 with heterogeneous (GPU / CPU) placement of parameter shards.

``HeteroDataParallel`` packs the model's parameters into chunks sharded over the DATA group; a module's chunks are
all-gathered right before it runs (forward and backward) and released afterwards, gradients are reduce-scattered
per chunk when backward is done with it.  ``placement_policy``: ``"cuda"`` keeps shards on the GPU, ``"cpu"`` in
pinned host memory, ``"auto"`` keeps them on the GPU while free device memory stays above ``min_free_fraction``.
``HeteroOptimizer`` runs the inner optimizer on fp32 master copies of the shards (on the shard's device, so CPU
shards are stepped by the host).  ``state_dict()`` gathers full tensors.

Parity: oslo/torch/nn/parallel/data_parallel/zero/hetero/{data_parallel,optim,memory_manager,placement_policy}.py
(the reference hard-codes fp16 there; any floating dtype works here).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from oslo_b200.distributed import ParallelMode
from oslo_b200.parallel.utils import ParallelWrapper, add_wrapper, get_parallel_context

from .chunk import Chunk, ChunkManager, search_chunk_size
from .memory_manager import MemoryManager, MemTracer


class MemStats:
    """Peak device memory and host<->device traffic observed per step (for the ``auto`` policy and for logs)."""

    def __init__(self):
        self.steps: List[dict] = []
        self.h2d_bytes = self.d2h_bytes = 0

    def record(self, **kw):
        self.steps.append(kw)


class PlacementPolicy:
    def __init__(self, name: str, compute_device, min_free_fraction: float = 0.2):
        if name not in ("cuda", "cpu", "auto", "const"):
            raise ValueError(f"unknown placement policy {name}")
        self.name, self.compute_device, self.min_free_fraction = name, compute_device, min_free_fraction

    def shard_device(self) -> torch.device:
        if self.name == "cpu" or self.compute_device.type == "cpu":
            return torch.device("cpu")
        if self.name in ("cuda", "const"):
            return self.compute_device
        free, total = torch.cuda.mem_get_info(self.compute_device)
        return self.compute_device if free / total > self.min_free_fraction else torch.device("cpu")


class HeteroDataParallel(ParallelWrapper):
    parallelism_priority = 99

    def __init__(self, module: nn.Module, parallel_context=None, placement_policy: str = "cuda", chunk_size_mb: Optional[float] = None,
                 pin_memory: bool = True, min_free_fraction: float = 0.2, device_budget_bytes: Optional[int] = None,
                 memory_probe=None, warmup_steps: int = 1):
        super().__init__()
        self.module = module
        self.parallel_context = pc = get_parallel_context(module, parallel_context)
        self.world = pc.get_world_size(ParallelMode.DATA)
        self.rank = pc.get_local_rank(ParallelMode.DATA)
        self.policy_name, self.chunk_size_mb, self.min_free_fraction = placement_policy, chunk_size_mb, min_free_fraction
        self.manager: Optional[ChunkManager] = None
        self.mem_stats = MemStats()
        # run-time placement ("auto"): budget of device bytes, probe of the device memory in use, traced warm-up steps
        self.device_budget_bytes, self.memory_probe, self.warmup_steps = device_budget_bytes, memory_probe, warmup_steps
        self.memory_manager: Optional[MemoryManager] = None
        self._hooks = []
        add_wrapper(module, ParallelMode.DATA, self)

    def parallelize(self):
        pc = self.parallel_context
        dev = pc.device
        for p in self.module.parameters():
            if p.device != dev:
                p.data = p.data.to(dev)
        params = [p for p in self.module.parameters() if p.requires_grad]
        if self.world > 1:
            src = pc.get_ranks_in_group(ParallelMode.DATA)[0]
            for p in params:
                dist.broadcast(p.data, src=src, group=pc.get_group(ParallelMode.DATA))
        policy = PlacementPolicy(self.policy_name, dev, self.min_free_fraction)
        esz = params[0].element_size() if params else 2
        if self.chunk_size_mb:
            unit = self.world * 128
            size = max(unit, int(self.chunk_size_mb * 2**20 / esz) // unit * unit)
            size = max(size, (max(p.numel() for p in params) + unit - 1) // unit * unit)
        else:
            size = search_chunk_size([p.numel() for p in params], self.world, elem_bytes=esz)
        self.manager = ChunkManager(self.world, self.rank, pc.get_group(ParallelMode.DATA), dev, policy.shard_device(), size)
        self.manager.register(params)
        if self.policy_name == "auto":
            for c in self.manager.chunks:  # under "auto" shards start on the device (logically, on a CPU-only run)
                c.on_device = True
            self.memory_manager = MemoryManager(self.manager.chunks, dev, self.device_budget_bytes, self.memory_probe,
                                                self.mem_stats, self.warmup_steps)
            self.manager.before_access = self.memory_manager.adjust_layout
        covered = set()  # modules inside a subtree that is gathered as one unit
        for m in self.module.modules():
            if id(m) in covered:
                continue
            subtree = getattr(m, "reads_descendant_parameters", False)
            if subtree:
                # the module's forward reads its descendants' parameters without calling them (fused ops over several
                # layers' weights): gather / release everything below it around ITS forward and backward
                covered.update(id(d) for d in m.modules() if d is not m)
            own = [p for p in m.parameters(recurse=subtree) if id(p) in self.manager.param_to_chunk]
            if not own:
                continue
            chunks = self.manager.chunks_of(own)
            self._hooks.append(m.register_forward_pre_hook(lambda mod, inp, c=chunks: self.manager.access(c)))
            self._hooks.append(m.register_forward_hook(lambda mod, inp, out, c=chunks: self._after_forward(c, mod, out)))
            self._hooks.append(m.register_full_backward_pre_hook(lambda mod, gout, c=chunks: self.manager.access(c)))
        for p in params:
            p.register_post_accumulate_grad_hook(self._grad_ready)
        for c in self.manager.chunks:
            c.pending_grads = len(c.params)

    def _after_forward(self, chunks, mod=None, out=None):
        """Release the module's chunks (modules re-gather on demand, so releasing is always safe).  A parameter that the
        module hands to its caller (``skip_bias_add`` layers return ``(output, bias)`` and the bias is added later, fused
        with dropout and the residual) must outlive the release: the caller gets a differentiable copy instead."""
        replaced = None
        if isinstance(out, tuple) and any(isinstance(o, nn.Parameter) for o in out):
            replaced = tuple(o.clone() if isinstance(o, nn.Parameter) else o for o in out)
        self.manager.release(chunks)
        return replaced

    def _grad_ready(self, p):
        c = self.manager.param_to_chunk[id(p)]
        c.pending_grads -= 1
        if c.pending_grads == 0:
            c.reduce_grads()
            c.release()
            c.pending_grads = len(c.params)

    def forward(self, *args, **kwargs):
        return self.module(*args, **kwargs)

    def backward(self, loss):
        loss.backward()
        self._flush_partial_chunks()

    def _flush_partial_chunks(self):
        """Chunks where some parameters got no gradient this step still have to be reduced."""
        for c in self.manager.chunks:
            if c.pending_grads != len(c.params):
                c.reduce_grads()
                c.release()
                c.pending_grads = len(c.params)

    def end_step(self):
        """Called by the optimizer after its update: lets the memory manager close the step (freeze the traced
        schedule after the warm-up, bring shards back to the device where they fit)."""
        if self.memory_manager is not None:
            self.memory_manager.end_step()

    def zero_grad(self, set_to_none=True):
        for c in self.manager.chunks:
            c.grad_shard = None
        for p in self.module.parameters():
            p.grad = None

    def state_dict(self, *args, **kwargs) -> Dict[str, torch.Tensor]:
        """Full (gathered) tensors, on the CPU."""
        out = {}
        names = {id(p): n for n, p in self.module.named_parameters()}
        for c in self.manager.chunks:
            was = c.is_gathered
            c.access()
            for p, off in zip(c.params, c.offsets):
                out[names[id(p)]] = c.full[off : off + p.oslo_numel].view(p.oslo_shape).detach().cpu().clone()
            if not was:
                c.release()
        for n, b in self.module.named_buffers():
            out[n] = b.detach().cpu()
        return out

    def load_state_dict(self, state: Dict[str, torch.Tensor], strict: bool = True):
        names = {id(p): n for n, p in self.module.named_parameters()}
        for c in self.manager.chunks:
            full = torch.zeros(c.size, dtype=c.dtype)
            for p, off in zip(c.params, c.offsets):
                full[off : off + p.oslo_numel].copy_(state[names[id(p)]].reshape(-1))
            lo = c.rank * c.shard_size
            c.shard.copy_(full[lo : lo + c.shard_size])
            c.write_back()

    def deparallelize(self):
        for h in self._hooks:
            h.remove()
        for c in self.manager.chunks:
            c.keep_gathered = True
            c.access()


class HeteroOptimizer:
    def __init__(self, model: HeteroDataParallel, optimizer: torch.optim.Optimizer, clip_grad_norm: float = 0.0, **unused):
        self.model, self.optim, self.clip_grad_norm = model, optimizer, clip_grad_norm
        self._built = False

    def _build(self):
        mgr = self.model.manager
        self.masters = [torch.nn.Parameter(c.shard.detach().float().clone()) for c in mgr.chunks]
        hyper = {k: v for k, v in self.optim.param_groups[0].items() if k != "params"}
        self.optim.param_groups.clear()
        self.optim.state.clear()
        self.optim.add_param_group({"params": self.masters, **hyper})
        self._built = True

    @property
    def param_groups(self):
        return self.optim.param_groups

    def zero_grad(self, set_to_none=True):
        self.model.zero_grad()

    def backward(self, loss):
        self.model.backward(loss)

    @torch.no_grad()
    def step(self):
        if not self._built:
            self._build()
        mgr = self.model.manager
        self.model._flush_partial_chunks()
        sq = torch.zeros(1)
        for c, m in zip(mgr.chunks, self.masters):
            g = c.grad_shard if c.grad_shard is not None else torch.zeros_like(c.shard)
            m.grad = g.float().to(m.device)
            sq += float(m.grad.pow(2).sum())
        if self.clip_grad_norm > 0:
            t = sq.to(self.model.parallel_context.device)
            if mgr.world > 1:
                dist.all_reduce(t, group=mgr.group)
            norm = float(t.sqrt())
            if norm > self.clip_grad_norm:
                for m in self.masters:
                    m.grad.mul_(self.clip_grad_norm / (norm + 1e-6))
        self.optim.step()
        for c, m in zip(mgr.chunks, self.masters):
            c.shard.copy_(m.data.to(c.shard.dtype))
            c.write_back()
            c.grad_shard = None
        self.model.end_step()

    def state_dict(self):
        return self.optim.state_dict()

    def load_state_dict(self, sd):
        if not self._built:
            self._build()
        self.optim.load_state_dict(sd)


__all__ = ["HeteroDataParallel", "HeteroOptimizer", "ChunkManager", "Chunk", "PlacementPolicy", "MemStats", "MemoryManager",
           "MemTracer", "search_chunk_size"]
