"""Causal language modelling: documents joined by EOS and cut into fixed-length chunks; labels = inputs."""
from __future__ import annotations

from typing import Dict, List

import torch

from .data_base import BaseProcessor, _SPMixin, pad_sequences


class ProcessorForCausalLM(BaseProcessor):
    def __call__(self, examples):
        column = "text" if "text" in examples else next(iter(examples))
        out: Dict[str, List[List[int]]] = {"input_ids": []}
        eos = getattr(self._tokenizer, "eos_token_id", None)
        for text in examples[column]:
            self._buffer.extend(self._encode(text))
            if eos is not None:
                self._buffer.append(eos)
            while len(self._buffer) >= self._chunk_size:
                out["input_ids"].append(self._buffer[: self._chunk_size])
                self._buffer = self._buffer[self._chunk_size :]
        return out


class DataCollatorForCausalLM(_SPMixin):
    def __init__(self, processor: ProcessorForCausalLM, parallel_context=None, label_pad_token_id: int = -100):
        self.tokenizer = processor._tokenizer
        self.label_pad_token_id = label_pad_token_id
        self.pad_token_id = getattr(self.tokenizer, "pad_token_id", None)
        if self.pad_token_id is None:
            self.pad_token_id = getattr(self.tokenizer, "eos_token_id", 0) or 0
        self._init_sp(parallel_context)

    def __call__(self, features):
        seqs = [f["input_ids"] for f in features]
        mult = self.sp_size if self.sp_size > 1 else None
        ids = pad_sequences(seqs, self.pad_token_id, mult)
        mask = pad_sequences([[1] * len(s) for s in seqs], 0, mult)
        labels = ids.masked_fill(mask == 0, self.label_pad_token_id)
        return self._slice({"input_ids": ids, "attention_mask": mask, "labels": labels})
