"""General-purpose collators: stack equal-shaped features, or pad tokenizer outputs to a common length.

Parity: oslo/transformers/data/data_collator.py (``default_data_collator``, ``DataCollatorWithPadding``).  The padding
collator works on any tokenizer-like object with ``pad_token_id`` (and optionally ``padding_side``); it does not call into
the tokenizer, so plain lists of ids from the task processors are enough.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional

import numpy as np
import torch

from .tasks.data_base import pad_sequences

_LABEL_KEYS = ("label", "label_ids")


def _as_dict(feature) -> Dict[str, Any]:
    return feature if isinstance(feature, dict) else vars(feature)


def default_data_collator(features: List[Any], return_tensors: str = "pt") -> Dict[str, Any]:
    """Stack every non-``None``, non-string field of the features; ``label`` / ``label_ids`` become ``labels`` (long for
    integers, float for regression targets).  ``return_tensors``: ``"pt"`` (torch) or ``"np"`` (numpy)."""
    if return_tensors not in ("pt", "np"):
        raise ValueError("return_tensors must be 'pt' or 'np'")
    feats = [_as_dict(f) for f in features]
    first = feats[0]
    batch: Dict[str, Any] = {}
    for key in _LABEL_KEYS:
        if key in first and first[key] is not None:
            sample = first[key]
            sample = sample.item() if torch.is_tensor(sample) and sample.dim() == 0 else sample
            is_float = isinstance(sample, float) or (torch.is_tensor(sample) and sample.is_floating_point()) or (
                isinstance(sample, (list, tuple, np.ndarray)) and np.asarray(sample).dtype.kind == "f")
            batch["labels"] = torch.as_tensor(np.asarray([np.asarray(f[key]) for f in feats]),
                                              dtype=torch.float32 if is_float else torch.long)
            break
    for k, v in first.items():
        if k in _LABEL_KEYS or v is None or isinstance(v, str):
            continue
        if torch.is_tensor(v):
            batch[k] = torch.stack([f[k] for f in feats])
        else:
            batch[k] = torch.as_tensor(np.asarray([np.asarray(f[k]) for f in feats]))
    if return_tensors == "np":
        batch = {k: v.numpy() for k, v in batch.items()}
    return batch


class DataCollatorWithPadding:
    """Pad ``input_ids`` (pad id), ``attention_mask`` / ``token_type_ids`` / ``special_tokens_mask`` (0) and per-token
    ``labels`` (``label_pad_token_id``) to the longest feature, to ``max_length`` and / or to a multiple."""

    def __init__(self, tokenizer, padding: bool = True, max_length: Optional[int] = None, pad_to_multiple_of: Optional[int] = None,
                 label_pad_token_id: int = -100):
        self.tokenizer, self.padding, self.max_length = tokenizer, padding, max_length
        self.pad_to_multiple_of, self.label_pad_token_id = pad_to_multiple_of, label_pad_token_id
        self.pad_id = getattr(tokenizer, "pad_token_id", None)
        if self.pad_id is None:
            self.pad_id = getattr(tokenizer, "eos_token_id", None) or 0
        self.left = getattr(tokenizer, "padding_side", "right") == "left"

    def __call__(self, features: List[Dict[str, Any]]) -> Dict[str, torch.Tensor]:
        feats = [_as_dict(f) for f in features]
        batch: Dict[str, torch.Tensor] = {}
        if "attention_mask" not in feats[0] and "input_ids" in feats[0]:
            feats = [dict(f, attention_mask=[1] * len(f["input_ids"])) for f in feats]
        for k in feats[0]:
            vals = [f[k].tolist() if torch.is_tensor(f[k]) else f[k] for f in feats]
            target = "labels" if k in _LABEL_KEYS else k
            if not isinstance(vals[0], (list, tuple)):
                batch[target] = torch.as_tensor(vals)
                continue
            fill = self.pad_id if k == "input_ids" else (self.label_pad_token_id if target == "labels" else 0)
            if not self.padding:
                batch[target] = torch.as_tensor(vals)
                continue
            if self.max_length:
                vals = [v[: self.max_length] for v in vals]
            t = pad_sequences(vals, fill, self.pad_to_multiple_of, left=self.left)
            if self.max_length and t.shape[1] < self.max_length and self.padding == "max_length":
                extra = t.new_full((t.shape[0], self.max_length - t.shape[1]), fill)
                t = torch.cat([extra, t] if self.left else [t, extra], dim=1)
            batch[target] = t
        return batch


__all__ = ["default_data_collator", "DataCollatorWithPadding"]
