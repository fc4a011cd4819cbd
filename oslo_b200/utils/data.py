"""Data collators (parity: oslo/torch/utils/data/data_collators.py:8-60)."""
from __future__ import annotations

from typing import Dict, List

import torch

from oslo_b200.distributed import ParallelMode


class SequenceParallelCollator:
    """Pads every sequence field to a multiple of the sequence-parallel size and keeps this rank's slice."""

    def __init__(self, parallel_key, parallel_context, dim: int = 1, pad_token_id: int = 0, label_pad_id: int = -100):
        self.keys = [parallel_key] if isinstance(parallel_key, str) else list(parallel_key)
        self.pc, self.dim = parallel_context, dim
        self.pad_token_id, self.label_pad_id = pad_token_id, label_pad_id
        self.world = parallel_context.get_world_size(ParallelMode.SEQUENCE)
        self.rank = parallel_context.get_local_rank(ParallelMode.SEQUENCE)

    def __call__(self, batch: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        out = dict(batch)
        for key in self.keys:
            if key not in out:
                continue
            t = out[key]
            n = t.shape[self.dim]
            pad = (-n) % self.world
            if pad:
                shape = list(t.shape)
                shape[self.dim] = pad
                fill = self.label_pad_id if key == "labels" else (0 if key == "attention_mask" else self.pad_token_id)
                t = torch.cat([t, t.new_full(shape, fill)], dim=self.dim)
            out[key] = t.chunk(self.world, dim=self.dim)[self.rank].contiguous()
        return out
