"""``DistributedDataParallel``: gradient averaging over the DATA group, overlapped with backward.

Gradients live in flat buffers (see ``_flat.py``); the buffer is cut into buckets in *reverse* parameter order
(the order backward produces gradients), and a bucket's all-reduce is issued on the communication stream the
moment its last gradient has been accumulated.  ``ShardingStrategy`` selects ZeRO instead and then the factory
returns ``(module, optimizer)`` like the reference.

Parity: oslo/torch/nn/parallel/data_parallel/data_parallel.py:31-264, _reducer.py:15-116.
"""
from __future__ import annotations

from enum import Enum
from typing import List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from oslo_b200.distributed import ParallelMode
from oslo_b200.parallel.utils import ParallelWrapper, add_wrapper, get_parallel_context

from ._flat import FlatBuffer, group_by_dtype


class ShardingStrategy(Enum):
    SHARD_PARAM = 1       # ZeRO stage 1: optimizer state sharded, gradients all-reduced
    SHARD_GRAD_PARAM = 2  # ZeRO stage 2: gradients reduce-scattered as well
    HETERO_SHARD = 3      # chunk-based ZeRO-3 with CPU / GPU placement


class _Bucket:
    def __init__(self, flat: FlatBuffer, start: int, end: int):
        self.flat, self.start, self.end = flat, start, end
        self.slots = flat.slots_in(start, end)
        self.pending = 0
        self.work = None


class _DistributedDataParallel(ParallelWrapper):
    parallelism_priority = 99

    def __init__(self, module: nn.Module, parallel_context=None, bucket_cap_mb: float = 25.0,
                 rebuild_bucket: bool = True, process_group_mode: ParallelMode = ParallelMode.DATA):
        super().__init__()
        self.module = module
        self.parallel_context = get_parallel_context(module, parallel_context)
        self.mode = process_group_mode
        self.bucket_cap_mb = bucket_cap_mb
        self.dp_world_size = self.parallel_context.get_world_size(self.mode)
        self.flats: List[FlatBuffer] = []
        self.buckets: List[_Bucket] = []
        self._slot_to_buckets = {}
        self._callback_queued = False
        self._require_sync = True
        add_wrapper(module, ParallelMode.DATA, self)

    def forward(self, *args, **kwargs):
        return self.module(*args, **kwargs)

    def parallelize(self):
        """Flatten gradients and install the hooks (run by ``oslo_b200.ready`` after TP / EP sharding)."""
        pc = self.parallel_context
        # expert weights are not replicated over DATA; row-sharded (ZeRO-3 style) linears reduce their own gradients
        skip = lambda p: getattr(p, "oslo_expert_param", False) or getattr(p, "oslo_zero_sharded", False)
        params = [p for p in self.module.parameters() if p.requires_grad and not skip(p)]
        if self.dp_world_size > 1:
            src = pc.get_ranks_in_group(self.mode)[0]
            for p in params:
                dist.broadcast(p.data, src=src, group=pc.get_group(self.mode))
        for (dtype, device), ps in group_by_dtype(params).items():
            flat = FlatBuffer(ps, pad_to=1, with_grads=True, flatten_params=False)
            self.flats.append(flat)
            esz = torch.empty((), dtype=dtype).element_size()
            cap = int(self.bucket_cap_mb * 1024 * 1024 / esz)
            for start, end in reversed(flat.bucket_ranges(cap)):
                b = _Bucket(flat, start, end)
                self.buckets.append(b)
                for s in b.slots:
                    self._slot_to_buckets.setdefault(id(s.param), []).append(b)
        for p in params:
            p.register_post_accumulate_grad_hook(self._hook)
        self._reset()

    def deparallelize(self):
        pass

    def _reset(self):
        for b in self.buckets:
            b.pending = len(b.slots)
            b.work = None

    def no_sync(self):
        """Context manager that skips gradient synchronisation (gradient accumulation micro-steps)."""
        wrapper = self

        class _NoSync:
            def __enter__(self):
                wrapper._require_sync = False

            def __exit__(self, *exc):
                wrapper._require_sync = True

        return _NoSync()

    def zero_grad(self, set_to_none: bool = False):
        for flat in self.flats:
            flat.zero_grad()

    def _hook(self, p):
        if not self._require_sync or self.dp_world_size == 1:
            return
        if not self._callback_queued:
            self._callback_queued = True
            torch.autograd.Variable._execution_engine.queue_callback(self._finish)
        for b in self._slot_to_buckets.get(id(p), ()):
            b.pending -= 1
            if b.pending == 0:
                self._launch(b)

    def _launch(self, b: _Bucket):
        pc = self.parallel_context
        group = pc.get_group(self.mode)
        view = b.flat.grad[b.start : b.end]
        # gradients may have been re-pointed by the user (zero_grad(set_to_none=True)): copy them back in
        for s in b.slots:
            g = s.param.grad
            if g is not None and g.data_ptr() != b.flat.grad[s.offset : s.offset + s.numel].data_ptr():
                b.flat.grad[s.offset : s.offset + s.numel].copy_(g.reshape(-1))
                s.param.grad = b.flat.grad[s.offset : s.offset + s.numel].view(s.param.shape)
        if dist.get_backend(group) == "nccl":
            b.work = dist.all_reduce(view, op=dist.ReduceOp.AVG, group=group, async_op=True)
        else:
            view.div_(self.dp_world_size)
            b.work = dist.all_reduce(view, group=group, async_op=True)

    def _finish(self):
        self._callback_queued = False
        for b in self.buckets:
            if b.work is None and b.pending != len(b.slots) and self._require_sync:
                self._launch(b)  # parameters that received no gradient this step
            if b.work is not None:
                b.work.wait()
        self._reset()


def DistributedDataParallel(module: nn.Module, parallel_context=None, model_wrapper_config: Optional[dict] = None,
                            optimizer_wrapper_config: Optional[dict] = None,
                            sharding_strategy: Optional[ShardingStrategy] = None, optimizer=None):
    """Wrap ``module`` for data parallelism; with a ``sharding_strategy`` also wrap ``optimizer`` in ZeRO and
    return ``(module, optimizer)``."""
    model_wrapper_config = model_wrapper_config or {}
    optimizer_wrapper_config = dict(optimizer_wrapper_config or {})
    if sharding_strategy is None:
        return _DistributedDataParallel(module, parallel_context, **model_wrapper_config)
    if optimizer is None:
        raise ValueError("a sharding_strategy needs the optimizer to shard")
    pc = get_parallel_context(module, parallel_context)
    if sharding_strategy == ShardingStrategy.HETERO_SHARD:
        from .zero.hetero import HeteroDataParallel, HeteroOptimizer

        wrapped = HeteroDataParallel(module, pc, **model_wrapper_config)
        return wrapped, HeteroOptimizer(wrapped, optimizer, **optimizer_wrapper_config)
    from .zero.optim import ZeroRedundancyOptimizer

    optimizer_wrapper_config["partition_grad"] = sharding_strategy == ShardingStrategy.SHARD_GRAD_PARAM
    module.parallel_context = pc
    return module, ZeroRedundancyOptimizer(optimizer, parallel_context=pc, **optimizer_wrapper_config)
