"""Sequence classification, token classification and summarisation processors / collators."""
from __future__ import annotations

import torch

from .data_base import BaseProcessor, _SPMixin, pad_sequences


class ProcessorForSequenceClassification(BaseProcessor):
    def __call__(self, examples):
        texts = examples["text"]
        out = {"input_ids": [], "labels": list(examples["labels"])}
        for t in texts:
            out["input_ids"].append(self._encode(t)[: self._max_length])
        return out


class DataCollatorForSequenceClassification(_SPMixin):
    def __init__(self, processor, parallel_context=None):
        self.tokenizer = processor._tokenizer
        self._init_sp(parallel_context)

    def __call__(self, features):
        pad = getattr(self.tokenizer, "pad_token_id", 0) or 0
        mult = self.sp_size if self.sp_size > 1 else None
        seqs = [f["input_ids"] for f in features]
        batch = {"input_ids": pad_sequences(seqs, pad, mult), "attention_mask": pad_sequences([[1] * len(s) for s in seqs], 0, mult)}
        batch = self._slice(batch)
        batch["labels"] = torch.as_tensor([f["labels"] for f in features])
        return batch


class ProcessorForTokenClassification(BaseProcessor):
    """Examples carry pre-split ``tokens`` and per-token ``labels``; sub-word pieces after the first get -100."""

    def __call__(self, examples):
        out = {"input_ids": [], "labels": []}
        for words, tags in zip(examples["tokens"], examples["labels"]):
            ids, labs = [], []
            for w, t in zip(words, tags):
                pieces = self._encode(w)
                ids += pieces
                labs += [t] + [-100] * (len(pieces) - 1)
            out["input_ids"].append(ids[: self._max_length])
            out["labels"].append(labs[: self._max_length])
        return out


class DataCollatorForTokenClassification(_SPMixin):
    def __init__(self, processor, parallel_context=None, label_pad_token_id: int = -100):
        self.tokenizer = processor._tokenizer
        self.label_pad_token_id = label_pad_token_id
        self._init_sp(parallel_context)

    def __call__(self, features):
        pad = getattr(self.tokenizer, "pad_token_id", 0) or 0
        mult = self.sp_size if self.sp_size > 1 else None
        seqs = [f["input_ids"] for f in features]
        return self._slice({"input_ids": pad_sequences(seqs, pad, mult),
                            "attention_mask": pad_sequences([[1] * len(s) for s in seqs], 0, mult),
                            "labels": pad_sequences([f["labels"] for f in features], self.label_pad_token_id, mult)})


class ProcessorForSummarization(BaseProcessor):
    def __init__(self, tokenizer, max_length: int = 512, max_target_length: int = 128):
        super().__init__(tokenizer, max_length)
        self._max_target_length = max_target_length

    def __call__(self, examples):
        out = {"input_ids": [], "labels": []}
        eos = getattr(self._tokenizer, "eos_token_id", None)
        for doc, summ in zip(examples["text"], examples["summary"]):
            out["input_ids"].append(self._encode(doc)[: self._max_length])
            lab = self._encode(summ)[: self._max_target_length - 1]
            out["labels"].append(lab + ([eos] if eos is not None else []))
        return out


class DataCollatorForSummarization(_SPMixin):
    def __init__(self, processor, parallel_context=None, label_pad_token_id: int = -100, decoder_start_token_id: int = None):
        self.tokenizer = processor._tokenizer
        self.label_pad_token_id = label_pad_token_id
        self.decoder_start_token_id = decoder_start_token_id
        self._init_sp(parallel_context)

    def __call__(self, features):
        pad = getattr(self.tokenizer, "pad_token_id", 0) or 0
        seqs = [f["input_ids"] for f in features]
        labels = pad_sequences([f["labels"] for f in features], self.label_pad_token_id)
        batch = {"input_ids": pad_sequences(seqs, pad), "attention_mask": pad_sequences([[1] * len(s) for s in seqs], 0), "labels": labels}
        start = self.decoder_start_token_id if self.decoder_start_token_id is not None else pad
        dec = labels.new_full(labels.shape, pad)
        dec[:, 1:] = labels[:, :-1].masked_fill(labels[:, :-1] == self.label_pad_token_id, pad)
        dec[:, 0] = start
        batch["decoder_input_ids"] = dec
        return batch
