"""Activation checkpointing with tensor-parallel partitioning of the saved activations.

``ActivationCheckpointing(module, parallel_context, partitioned_checkpointing, contiguous_checkpointing,
cpu_checkpointing)`` turns on gradient checkpointing for the model and makes every checkpointed region use
:class:`CheckpointFunction`, which

* saves and restores the RNG state (CPU, device and the per-``ParallelMode`` seed manager) so dropout replays,
* with ``partitioned_checkpointing`` keeps only ``1/tp`` of every saved input on each tensor-parallel rank and
  all-gathers it back right before the recomputation,
* with ``cpu_checkpointing`` parks the kept part in pinned host memory,
* with ``contiguous_checkpointing`` packs the kept parts of one region into one buffer.

Parity: oslo/torch/utils/checkpoint/activation_checkpointing.py:37-97, _checkpoint_function.py:13-187,
_checkpoint_partitioner.py:10-260, _rng_state_tracker.py:10-109.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.utils.checkpoint as torch_checkpoint

from oslo_b200.distributed import ParallelMode, comm
from oslo_b200.distributed import seed as seed_mod


class CheckpointPartitioner:
    """Splits saved activations over the tensor group and restores them."""

    def __init__(self, parallel_context=None, partitioned=False, contiguous=False, cpu=False):
        self.pc = parallel_context
        self.partitioned = partitioned and parallel_context is not None and parallel_context.tensor_parallel_size > 1
        self.contiguous, self.cpu = contiguous, cpu

    def _tp(self):
        return self.pc.get_world_size(ParallelMode.TENSOR), self.pc.get_local_rank(ParallelMode.TENSOR)

    def partition(self, tensors: List[Optional[torch.Tensor]]):
        """Returns ``(kept, meta)``: what stays resident and what is needed to rebuild the originals."""
        kept, meta = [], []
        for t in tensors:
            if not torch.is_tensor(t) or not t.is_floating_point():
                kept.append(t)
                meta.append(None)
                continue
            shape, dev = t.shape, t.device
            part = t.detach()
            padded = 0
            if self.partitioned:
                world, rank = self._tp()
                flat = part.reshape(-1)
                padded = (-flat.numel()) % world
                if padded:
                    flat = torch.cat([flat, flat.new_zeros(padded)])
                part = flat.chunk(world)[rank].clone()
            if self.cpu and part.is_cuda:
                host = torch.empty(part.shape, dtype=part.dtype, pin_memory=True)
                host.copy_(part, non_blocking=True)
                part = host
            kept.append(part)
            meta.append((shape, dev, padded, t.requires_grad))
        if self.contiguous:
            floats = [(i, k) for i, (k, m) in enumerate(zip(kept, meta)) if m is not None]
            if floats and all(k.dtype == floats[0][1].dtype and k.device == floats[0][1].device for _, k in floats):
                buf = torch.cat([k.reshape(-1) for _, k in floats])
                off = 0
                for i, k in floats:
                    kept[i] = buf[off : off + k.numel()].view(k.shape)
                    off += k.numel()
        return kept, meta

    def restore(self, kept, meta):
        out = []
        for k, m in zip(kept, meta):
            if m is None:
                out.append(k)
                continue
            shape, dev, padded, requires_grad = m
            t = k.to(dev, non_blocking=True) if k.device != dev else k
            if self.partitioned:
                t = comm.all_gather(t.contiguous(), dim=0, parallel_context=self.pc, parallel_mode=ParallelMode.TENSOR)
                if padded:
                    t = t[: t.numel() - padded]
            t = t.reshape(shape).detach()
            t.requires_grad_(requires_grad)
            out.append(t)
        return out


class CudaRNGStatesTracker:
    """Named RNG states with a ``fork`` context manager (device generator when CUDA is up, CPU otherwise)."""

    def __init__(self):
        self.states, self.seeds = {}, set()

    def reset(self):
        self.states, self.seeds = {}, set()

    def get_states(self):
        return dict(self.states)

    def set_states(self, states):
        self.states = dict(states)

    def add(self, name, seed):
        if seed in self.seeds or name in self.states:
            raise RuntimeError(f"seed {seed} / state {name} already registered")
        self.seeds.add(seed)
        orig = seed_mod._get_state()
        seed_mod._manual_seed(seed)
        self.states[name] = seed_mod._get_state()
        seed_mod._set_state(orig)

    def fork(self, name="model-parallel-rng"):
        tracker = self

        class _Fork:
            def __enter__(self):
                self.orig = seed_mod._get_state()
                seed_mod._set_state(tracker.states[name])

            def __exit__(self, *exc):
                tracker.states[name] = seed_mod._get_state()
                seed_mod._set_state(self.orig)

        return _Fork()


_partitioner = CheckpointPartitioner()


class CheckpointFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, run_function, partitioner, *args):
        ctx.run_function, ctx.partitioner = run_function, partitioner
        ctx.cpu_rng = torch.get_rng_state()
        ctx.dev_rng = torch.cuda.get_rng_state() if torch.cuda.is_available() and torch.cuda.is_initialized() else None
        ctx.seed_states = seed_mod.get_states(copy=True)
        ctx.seed_mode = seed_mod.get_current_mode()
        with torch.no_grad():
            outputs = run_function(*args)
        kept, meta = partitioner.partition(list(args))
        ctx.meta = meta
        ctx.tensor_idx = [i for i, k in enumerate(kept) if torch.is_tensor(k)]
        ctx.others = [None if torch.is_tensor(k) else k for k in kept]
        ctx.save_for_backward(*[kept[i] for i in ctx.tensor_idx])
        return outputs

    @staticmethod
    def backward(ctx, *grads):
        kept = list(ctx.others)
        for i, t in zip(ctx.tensor_idx, ctx.saved_tensors):
            kept[i] = t
        inputs = ctx.partitioner.restore(kept, ctx.meta)
        now_cpu = torch.get_rng_state()
        now_dev = torch.cuda.get_rng_state() if ctx.dev_rng is not None else None
        now_seed = seed_mod.get_states(copy=True)
        torch.set_rng_state(ctx.cpu_rng)
        if ctx.dev_rng is not None:
            torch.cuda.set_rng_state(ctx.dev_rng)
        for mode, state in ctx.seed_states.items():
            seed_mod.set_seed_states(mode, state)
        with torch.enable_grad():
            outputs = ctx.run_function(*inputs)
        torch.set_rng_state(now_cpu)
        if now_dev is not None:
            torch.cuda.set_rng_state(now_dev)
        for mode, state in now_seed.items():
            seed_mod.set_seed_states(mode, state)
        if torch.is_tensor(outputs):
            outputs = (outputs,)
        pairs = [(o, g) for o, g in zip(outputs, grads) if torch.is_tensor(o) and o.requires_grad and g is not None]
        torch.autograd.backward([o for o, _ in pairs], [g for _, g in pairs])
        return (None, None) + tuple(t.grad if torch.is_tensor(t) and t.requires_grad else None for t in inputs)


def checkpoint(function, *args, partitioner: Optional[CheckpointPartitioner] = None, **kwargs):
    """Drop-in for ``torch.utils.checkpoint.checkpoint`` (keyword-only extras such as ``use_reentrant`` are accepted)."""
    return CheckpointFunction.apply(function, partitioner or _partitioner, *args)


class ActivationCheckpointing:
    def __init__(self, module, parallel_context=None, partitioned_checkpointing=False, contiguous_checkpointing=False,
                 cpu_checkpointing=False):
        global _partitioner
        self.module = module
        self.partitioner = CheckpointPartitioner(parallel_context, partitioned_checkpointing, contiguous_checkpointing,
                                                 cpu_checkpointing)
        _partitioner = self.partitioner
        part = self.partitioner

        def patched(function, *args, **kwargs):
            return CheckpointFunction.apply(function, part, *args)

        # regions inside the model call torch.utils.checkpoint.checkpoint: route them here
        self._orig = torch_checkpoint.checkpoint
        torch_checkpoint.checkpoint = patched
        torch.utils.checkpoint.checkpoint = patched
        base = module
        while hasattr(base, "module") and not hasattr(base, "gradient_checkpointing_enable"):
            base = base.module
        if hasattr(base, "gradient_checkpointing_enable"):
            base.gradient_checkpointing_enable()

    def disable(self):
        torch_checkpoint.checkpoint = self._orig
        torch.utils.checkpoint.checkpoint = self._orig
