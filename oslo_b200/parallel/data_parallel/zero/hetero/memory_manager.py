"""Run-time placement of ZeRO-3 parameter shards between device and (pinned) host memory.

The placement chosen when the model is wrapped is only a starting point.  During training the memory a step needs
besides parameters (activations, workspaces) changes from moment to moment; the ``auto`` policy keeps as many shards on
the device as fit *at every moment*:

* ``MemTracer`` samples, at every chunk access of a warm-up step, how much device memory is in use that is NOT chunk
  memory (``non_model``) and records the order in which chunks are needed (the compute schedule);
* before a chunk is gathered, ``MemoryManager.adjust_layout`` checks ``non_model (as traced at this moment) + resident
  shards + gathered buffers + the incoming buffer`` against the budget and, if it does not fit, moves resident shards
  of OTHER chunks to host memory, the one whose next use lies furthest in the future first (it is the cheapest to
  lose), exactly until the access fits;
* after the step, shards are brought back to the device in order of next use while the traced peak leaves room.

Parity: oslo/torch/nn/parallel/data_parallel/zero/hetero/memory_manager.py:39-255 (``adjust_layout``),
placement_policy.py:100-310 (``AutoPlacementPolicy.evict_tensors`` and the warm-up statistics), memory_tracer/*.
The budget and the "device memory in use" probe can be injected, which is how the logic is tested without a GPU.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional

import torch


class MemTracer:
    """Non-model device memory per access moment and the chunk access schedule of one (warm-up) step."""

    def __init__(self, probe: Callable[[], int]):
        self.probe = probe
        self.non_model: List[int] = []   # bytes in use besides chunk memory, one sample per access moment
        self.schedule: List[int] = []    # chunk index per access moment
        self.recording = True

    def sample(self, chunk_index: int, chunk_bytes_on_device: int):
        if not self.recording:
            return
        self.non_model.append(max(0, int(self.probe()) - int(chunk_bytes_on_device)))
        self.schedule.append(chunk_index)

    def finish(self):
        self.recording = False

    def non_model_at(self, moment: int) -> int:
        if not self.non_model:
            return 0
        return self.non_model[min(moment, len(self.non_model) - 1)]

    @property
    def peak_non_model(self) -> int:
        return max(self.non_model, default=0)


class MemoryManager:
    def __init__(self, chunks, compute_device, budget_bytes: Optional[int] = None, probe: Optional[Callable[[], int]] = None,
                 stats=None, warmup_steps: int = 1, pin_memory: bool = True):
        self.chunks = list(chunks)
        self.index: Dict[int, int] = {id(c): i for i, c in enumerate(self.chunks)}
        self.compute_device = compute_device
        if probe is None:
            if compute_device.type == "cuda":
                probe = lambda: torch.cuda.memory_allocated(compute_device)
            else:
                probe = lambda: 0
        if budget_bytes is None:
            if compute_device.type == "cuda":
                _, total = torch.cuda.mem_get_info(compute_device)
                budget_bytes = int(total * 0.8)
            else:
                budget_bytes = 1 << 62
        self.budget = int(budget_bytes)
        self.tracer = MemTracer(probe)
        self.stats = stats
        self.warmup_steps = warmup_steps
        self.pin_memory = pin_memory and torch.cuda.is_available()
        self.moment = 0
        self.step_no = 0
        self.evictions = 0
        self.promotions = 0
        self.peak_model_bytes = 0
        for c in self.chunks:
            if not hasattr(c, "on_device"):
                c.on_device = c.shard_device.type == compute_device.type and compute_device.type != "cpu"

    # ------------------------------------------------------------ accounting
    @staticmethod
    def _shard_bytes(c) -> int:
        return c.shard.numel() * c.shard.element_size()

    @staticmethod
    def _full_bytes(c) -> int:
        return c.size * torch.empty((), dtype=c.dtype).element_size()

    def model_bytes_on_device(self) -> int:
        total = 0
        for c in self.chunks:
            if c.on_device:
                total += self._shard_bytes(c)
            if c.full is not None:
                total += self._full_bytes(c)
        return total

    def _next_use(self, chunk_index: int) -> int:
        """Moments until ``chunk_index`` is needed again (a large number if not before the end of the step)."""
        sched = self.tracer.schedule
        for m in range(self.moment, len(sched)):
            if sched[m] == chunk_index:
                return m - self.moment
        return len(sched) + sched.index(chunk_index) if chunk_index in sched else 1 << 30

    # ---------------------------------------------------------------- moves
    def _to_host(self, c):
        if not c.on_device:
            return
        nbytes = self._shard_bytes(c)
        host = c.shard.to("cpu")
        if self.pin_memory:
            host = host.pin_memory()
        c.shard = host
        if c.grad_shard is not None:
            c.grad_shard = c.grad_shard.to("cpu")
        c.shard_device = torch.device("cpu")
        c.on_device = False
        self.evictions += 1
        if self.stats is not None:
            self.stats.d2h_bytes += nbytes

    def _to_device(self, c):
        if c.on_device:
            return
        nbytes = self._shard_bytes(c)
        c.shard = c.shard.to(self.compute_device, non_blocking=True)
        if c.grad_shard is not None:
            c.grad_shard = c.grad_shard.to(self.compute_device)
        c.shard_device = self.compute_device
        c.on_device = True
        self.promotions += 1
        if self.stats is not None:
            self.stats.h2d_bytes += nbytes

    # ------------------------------------------------------------ the policy
    def adjust_layout(self, chunk) -> None:
        """Called right before ``chunk`` is gathered to the compute device."""
        ci = self.index[id(chunk)]
        model = self.model_bytes_on_device()
        if self.tracer.recording:
            self.tracer.sample(ci, model)
        need = 0 if chunk.full is not None else self._full_bytes(chunk)
        non_model = self.tracer.non_model_at(self.moment) if not self.tracer.recording else self.tracer.non_model[-1]
        over = non_model + model + need - self.budget
        if over > 0:
            victims = [c for c in self.chunks if c.on_device and c is not chunk and c.full is None]
            victims.sort(key=lambda c: self._next_use(self.index[id(c)]), reverse=True)
            for v in victims:
                if over <= 0:
                    break
                over -= self._shard_bytes(v)
                self._to_host(v)
        self.peak_model_bytes = max(self.peak_model_bytes, self.model_bytes_on_device() + need)
        self.moment += 1

    def end_step(self) -> None:
        """Close the step: after the warm-up the schedule is frozen; then bring shards back while they fit under the
        traced peak of everything else."""
        self.step_no += 1
        if self.tracer.recording and self.step_no >= self.warmup_steps:
            self.tracer.finish()
        self.moment = 0
        if self.tracer.recording:
            return
        largest = max((self._full_bytes(c) for c in self.chunks), default=0)
        room = self.budget - self.tracer.peak_non_model - self.model_bytes_on_device() - 2 * largest
        order = sorted((c for c in self.chunks if not c.on_device), key=lambda c: self._next_use(self.index[id(c)]))
        for c in order:
            n = self._shard_bytes(c)
            if n > room:
                break
            self._to_device(c)
            room -= n
