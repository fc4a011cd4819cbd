"""Processors and collators for the pre-training / fine-tuning tasks.

A *processor* turns a batch of raw examples (``{"text": [...]}``) into model-ready lists through
``datasets.map(processor, batched=True)``-style calls; a *collator* pads a list of features into tensors, optionally
padding to a multiple (e.g. of the sequence-parallel size) and slicing this rank's part.  Tokenizers are duck-typed:
anything with ``__call__`` returning ``input_ids`` lists and the usual ``*_token_id`` attributes works, so the Hugging
Face tokenizers plug in directly.  Parity: oslo/transformers/tasks/*.py.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional

import torch


class BaseProcessor:
    def __init__(self, tokenizer, max_length: int = 512):
        self._tokenizer = tokenizer
        self._max_length = max_length
        self._chunk_size = max_length
        self._buffer: List[int] = []

    def save_tokenizer(self, path: str) -> None:
        if hasattr(self._tokenizer, "save_pretrained"):
            self._tokenizer.save_pretrained(path)

    def _encode(self, text: str) -> List[int]:
        out = self._tokenizer(text, add_special_tokens=False) if callable(self._tokenizer) else self._tokenizer.encode(text)
        return out["input_ids"] if isinstance(out, dict) or hasattr(out, "keys") else list(out)

    def __call__(self, examples: Dict[str, List[Any]]) -> Dict[str, List[Any]]:
        raise NotImplementedError


def pad_sequences(seqs: List[List[int]], pad_value: int, pad_to_multiple_of: Optional[int] = None, left: bool = False) -> torch.Tensor:
    n = max(len(s) for s in seqs)
    if pad_to_multiple_of:
        n = (n + pad_to_multiple_of - 1) // pad_to_multiple_of * pad_to_multiple_of
    out = torch.full((len(seqs), n), pad_value, dtype=torch.long)
    for i, s in enumerate(seqs):
        if left:
            out[i, n - len(s):] = torch.as_tensor(s, dtype=torch.long)
        else:
            out[i, : len(s)] = torch.as_tensor(s, dtype=torch.long)
    return out


class _SPMixin:
    """Optional sequence-parallel slicing of every [batch, seq] tensor."""

    def _init_sp(self, parallel_context):
        self.parallel_context = parallel_context
        self.sp_size, self.sp_rank = 1, 0
        if parallel_context is not None:
            from oslo_b200.distributed import ParallelMode

            self.sp_size = parallel_context.get_world_size(ParallelMode.SEQUENCE)
            self.sp_rank = parallel_context.get_local_rank(ParallelMode.SEQUENCE)

    def _slice(self, batch: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        if self.sp_size == 1:
            return batch
        return {k: (v.chunk(self.sp_size, dim=1)[self.sp_rank].contiguous() if torch.is_tensor(v) and v.dim() >= 2 else v)
                for k, v in batch.items()}
