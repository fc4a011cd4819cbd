"""Flat parameter / gradient buffers shared by DDP and ZeRO.

Parameters of one dtype are laid out back to back (each start aligned to 128 elements) in one contiguous
buffer; ``p.data`` and ``p.grad`` become views into the flat buffers, so autograd accumulates gradients
directly into communication memory and no bucket copy-in / copy-out pass exists (the reference copies every
gradient into a 25 MB bucket and back: oslo/torch/nn/parallel/data_parallel/_reducer.py:30-116).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Sequence

import torch

ALIGN = 128  # elements


@dataclass
class Slot:
    param: torch.nn.Parameter
    offset: int
    numel: int


class FlatBuffer:
    """One contiguous buffer holding the given parameters (same dtype/device), padded to ``pad_to`` elements."""

    @staticmethod
    def layout_numel(params: Sequence[torch.nn.Parameter], pad_to: int = 1) -> int:
        """Elements the flat buffer will have for these parameters (to size externally provided storage)."""
        off = 0
        for p in params:
            off += (p.numel() + ALIGN - 1) // ALIGN * ALIGN
        total = (off + pad_to - 1) // pad_to * pad_to if pad_to > 1 else off
        return max(total, pad_to)

    def __init__(self, params: Sequence[torch.nn.Parameter], pad_to: int = 1, with_grads: bool = True, flatten_params: bool = True,
                 param_storage: torch.Tensor = None, grad_storage: torch.Tensor = None):
        self.dtype = params[0].dtype
        self.device = params[0].device
        self.slots: List[Slot] = []
        off = 0
        for p in params:
            self.slots.append(Slot(p, off, p.numel()))
            off += (p.numel() + ALIGN - 1) // ALIGN * ALIGN
        total = (off + pad_to - 1) // pad_to * pad_to if pad_to > 1 else off
        self.numel = max(total, pad_to)
        self.param = None
        if flatten_params:
            self.param = param_storage if param_storage is not None else torch.zeros(self.numel, dtype=self.dtype, device=self.device)
            assert self.param.numel() == self.numel and self.param.dtype == self.dtype
            for s in self.slots:
                view = self.param[s.offset : s.offset + s.numel].view(s.param.shape)
                view.copy_(s.param.data)
                s.param.data = view
        if with_grads:
            self.grad = grad_storage if grad_storage is not None else torch.zeros(self.numel, dtype=self.dtype, device=self.device)
            self.grad.zero_()
        else:
            self.grad = None
        if with_grads:
            self.attach_grads()

    def attach_grads(self):
        """Point every ``p.grad`` at its slice of the flat gradient buffer (call again after ``zero_grad(None)``)."""
        for s in self.slots:
            s.param.grad = self.grad[s.offset : s.offset + s.numel].view(s.param.shape)

    def zero_grad(self):
        self.grad.zero_()
        self.attach_grads()

    def bucket_ranges(self, bucket_elems: int, multiple: int = 1):
        """Split ``[0, numel)`` into consecutive ranges of about ``bucket_elems`` (each a multiple of ``multiple``)."""
        step = max(multiple, (bucket_elems + multiple - 1) // multiple * multiple)
        out = []
        start = 0
        while start < self.numel:
            end = min(self.numel, start + step)
            out.append((start, end))
            start = end
        return out

    def slots_in(self, start: int, end: int) -> List[Slot]:
        return [s for s in self.slots if s.offset < end and s.offset + s.numel > start]


def group_by_dtype(params) -> Dict[torch.dtype, List[torch.nn.Parameter]]:
    out: Dict[torch.dtype, List[torch.nn.Parameter]] = {}
    for p in params:
        if p.requires_grad:
            out.setdefault((p.dtype, p.device), []).append(p)
    return out
