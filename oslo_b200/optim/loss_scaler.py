"""Dynamic loss scaling for fp16 training.

The interface follows ``torch.amp.GradScaler`` (``scale`` / ``unscale_`` / ``step`` / ``update`` / ``state_dict``), which
is what the reference trainer drives (oslo/transformers/trainer.py:477-494,607,768,840 keep a ``scaler`` beside the
optimizer and save it as ``scaler.pt``).  Differences that matter for the parallel wrappers here:

* the overflow verdict is one fused pass: all gradients are reduced to a single non-finite flag with ``torch._foreach``
  norms (no per-tensor host sync), and the flag is all-reduced (MAX) over an optional process group, so tensor- /
  pipeline- / data-parallel ranks skip or take a step together;
* un-scaling multiplies by ``1 / scale`` in the same foreach pass, in place, and is idempotent per step;
* works on CPU tensors (tests, CPU-offloaded optimizers) as well as CUDA.

bf16 training does not need it (same exponent range as fp32): the trainer only builds a scaler for ``fp16=True``.
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Optional

import torch
import torch.distributed as dist


class DynamicLossScaler:
    def __init__(self, init_scale: float = 2.0 ** 16, growth_factor: float = 2.0, backoff_factor: float = 0.5,
                 growth_interval: int = 2000, min_scale: float = 1.0, max_scale: float = 2.0 ** 24, enabled: bool = True,
                 group=None):
        if growth_factor <= 1.0 or not 0.0 < backoff_factor < 1.0:
            raise ValueError("growth_factor must exceed 1 and backoff_factor lie in (0, 1)")
        self.enabled, self.group = enabled, group
        self._scale = float(init_scale) if enabled else 1.0
        self.growth_factor, self.backoff_factor, self.growth_interval = growth_factor, backoff_factor, growth_interval
        self.min_scale, self.max_scale = min_scale, max_scale
        self._good_steps = 0
        self._unscaled: Dict[int, bool] = {}  # id(optimizer) -> found_inf of this step
        self.skipped_steps = 0

    # ------------------------------------------------------------------ state
    def get_scale(self) -> float:
        return self._scale

    def state_dict(self) -> dict:
        return {"scale": self._scale, "good_steps": self._good_steps, "growth_factor": self.growth_factor,
                "backoff_factor": self.backoff_factor, "growth_interval": self.growth_interval, "skipped_steps": self.skipped_steps}

    def load_state_dict(self, sd: dict) -> None:
        self._scale = float(sd["scale"])
        self._good_steps = int(sd.get("good_steps", 0))
        self.growth_factor = sd.get("growth_factor", self.growth_factor)
        self.backoff_factor = sd.get("backoff_factor", self.backoff_factor)
        self.growth_interval = sd.get("growth_interval", self.growth_interval)
        self.skipped_steps = int(sd.get("skipped_steps", 0))

    # ------------------------------------------------------------------- flow
    def scale(self, loss: torch.Tensor) -> torch.Tensor:
        return loss * self._scale if self.enabled else loss

    @staticmethod
    def _grads(optimizer) -> List[torch.Tensor]:
        return [p.grad for g in optimizer.param_groups for p in g["params"] if p.grad is not None]

    def _found_inf(self, grads: Iterable[torch.Tensor]) -> bool:
        grads = list(grads)
        flag = None
        by_kind: Dict[tuple, List[torch.Tensor]] = {}
        for g in grads:
            by_kind.setdefault((g.device, g.dtype), []).append(g)
        for (device, _), gs in by_kind.items():
            # the sum of the per-tensor norms is non-finite iff any element is
            total = torch.stack(torch._foreach_norm(gs, 2.0)).float().sum()
            bad = (~torch.isfinite(total)).float().to(flag.device if flag is not None else device)
            flag = bad if flag is None else torch.maximum(flag, bad)
        if flag is None:
            flag = torch.zeros((), device="cpu")
        if self.group is not None and dist.is_initialized() and dist.get_world_size(self.group) > 1:
            flag = flag.reshape(1)
            dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=self.group)
        return bool(flag.item() > 0)

    def unscale_(self, optimizer) -> bool:
        """Divide the optimizer's gradients by the scale (once per step) and return whether any is non-finite."""
        key = id(optimizer)
        if key in self._unscaled:
            return self._unscaled[key]
        grads = self._grads(optimizer)
        found = False
        if self.enabled:
            found = self._found_inf(grads)
            if not found and grads and self._scale != 1.0:
                torch._foreach_mul_(grads, 1.0 / self._scale)
        self._unscaled[key] = found
        return found

    def step(self, optimizer, *args, **kwargs):
        """``optimizer.step()`` unless this step's gradients overflowed; returns its result (``None`` when skipped)."""
        found = self.unscale_(optimizer)
        if found:
            self.skipped_steps += 1
            return None
        return optimizer.step(*args, **kwargs)

    def update(self) -> None:
        """Shrink the scale after an overflow, grow it after ``growth_interval`` clean steps; forget this step's verdicts."""
        if self.enabled and self._unscaled:
            if any(self._unscaled.values()):
                self._scale = max(self._scale * self.backoff_factor, self.min_scale)
                self._good_steps = 0
            else:
                self._good_steps += 1
                if self._good_steps >= self.growth_interval:
                    self._scale = min(self._scale * self.growth_factor, self.max_scale)
                    self._good_steps = 0
        self._unscaled = {}


__all__ = ["DynamicLossScaler"]
