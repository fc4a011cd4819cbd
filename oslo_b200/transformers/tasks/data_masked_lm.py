"""Masked language modelling (BERT / RoBERTa style dynamic masking: 80 % [MASK], 10 % random, 10 % kept)."""
from __future__ import annotations

import torch

from .data_base import BaseProcessor, _SPMixin, pad_sequences


class ProcessorForMaskedLM(BaseProcessor):
    def __init__(self, tokenizer, max_length: int = 512):
        super().__init__(tokenizer, max_length)
        self._chunk_size = max_length - 2  # room for [CLS] ... [SEP]

    def __call__(self, examples):
        column = "text" if "text" in examples else next(iter(examples))
        cls_id = getattr(self._tokenizer, "cls_token_id", None)
        sep_id = getattr(self._tokenizer, "sep_token_id", None)
        out = {"input_ids": []}
        for text in examples[column]:
            self._buffer.extend(self._encode(text))
            while len(self._buffer) >= self._chunk_size:
                chunk = self._buffer[: self._chunk_size]
                self._buffer = self._buffer[self._chunk_size :]
                if cls_id is not None and sep_id is not None:
                    chunk = [cls_id] + chunk + [sep_id]
                out["input_ids"].append(chunk)
        return out


class DataCollatorForMaskedLM(_SPMixin):
    def __init__(self, processor, mlm_probability: float = 0.15, parallel_context=None, label_pad_token_id: int = -100, seed: int = None):
        self.tokenizer = processor._tokenizer
        self.mlm_probability = mlm_probability
        self.label_pad_token_id = label_pad_token_id
        self.generator = torch.Generator()
        if seed is not None:
            self.generator.manual_seed(seed)
        self._init_sp(parallel_context)

    def _special_mask(self, ids):
        special = torch.zeros_like(ids, dtype=torch.bool)
        for name in ("cls_token_id", "sep_token_id", "pad_token_id", "bos_token_id", "eos_token_id"):
            tid = getattr(self.tokenizer, name, None)
            if tid is not None:
                special |= ids == tid
        return special

    def mask_tokens(self, ids):
        labels = ids.clone()
        prob = torch.full(ids.shape, self.mlm_probability)
        prob.masked_fill_(self._special_mask(ids), 0.0)
        masked = torch.bernoulli(prob, generator=self.generator).bool()
        labels[~masked] = self.label_pad_token_id
        ids = ids.clone()
        replace = torch.bernoulli(torch.full(ids.shape, 0.8), generator=self.generator).bool() & masked
        ids[replace] = self.tokenizer.mask_token_id
        rand = torch.bernoulli(torch.full(ids.shape, 0.5), generator=self.generator).bool() & masked & ~replace
        vocab = getattr(self.tokenizer, "vocab_size", None) or len(self.tokenizer)
        ids[rand] = torch.randint(vocab, ids.shape, generator=self.generator)[rand]
        return ids, labels

    def __call__(self, features):
        pad = getattr(self.tokenizer, "pad_token_id", 0) or 0
        mult = self.sp_size if self.sp_size > 1 else None
        seqs = [f["input_ids"] for f in features]
        ids = pad_sequences(seqs, pad, mult)
        mask = pad_sequences([[1] * len(s) for s in seqs], 0, mult)
        ids, labels = self.mask_tokens(ids)
        labels = labels.masked_fill(mask == 0, self.label_pad_token_id)
        return self._slice({"input_ids": ids, "attention_mask": mask, "labels": labels})
