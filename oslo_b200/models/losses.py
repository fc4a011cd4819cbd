"""Next-token loss shared by the in-tree causal LMs.

Picks the loss class from the tensor-parallel mode like the reference's GPT-2
(oslo/transformers/models/gpt2/modeling_gpt2.py:845-875): vocab-parallel cross-entropy for 1D / 2D / 2.5D,
plain cross-entropy on gathered logits for 3D and for an unsharded model.  The shift by one position is done
on the labels (``labels[:, 1:]`` padded with ``ignore_index``) so the logits are never sliced or copied.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F

import oslo_b200.nn as onn
from oslo_b200.distributed import ParallelMode


@dataclass
class LossResult:
    value: torch.Tensor
    consumed_logits: bool


def shift_labels(labels: torch.Tensor, ignore_index: int = -100) -> torch.Tensor:
    out = torch.full_like(labels, ignore_index)
    out[..., :-1] = labels[..., 1:]
    return out


def causal_lm_loss(model, logits, labels, ignore_index: int = -100) -> LossResult:
    return token_lm_loss(model, logits, shift_labels(labels, ignore_index), ignore_index)


def token_lm_loss(model, logits, targets, ignore_index: int = -100) -> LossResult:
    """Cross-entropy of ``logits[..., t, :]`` against ``targets[..., t]`` (masked-LM and sequence-to-sequence heads use it
    directly; the causal heads shift the labels first)."""
    pc = getattr(model, "parallel_context", None)
    sharded_vocab = logits.shape[-1] != getattr(model, "padded_vocab_size", model.config.vocab_size) \
        and logits.shape[-1] != model.config.vocab_size
    mode = pc.tensor_parallel_mode if pc is not None else None
    orig_vocab = model.config.vocab_size
    if pc is not None and sharded_vocab and mode in (ParallelMode.TENSOR_1D, ParallelMode.TENSOR_2D, ParallelMode.TENSOR_2P5D):
        cls = {ParallelMode.TENSOR_1D: onn.VocabParallelCrossEntropyLoss1D,
               ParallelMode.TENSOR_2D: onn.VocabParallelCrossEntropyLoss2D,
               ParallelMode.TENSOR_2P5D: onn.VocabParallelCrossEntropyLoss2p5D}[mode]
        fn = cls(parallel_context=pc, ignore_index=ignore_index)
        fn.orig_vocab_size = orig_vocab
        return LossResult(fn(logits, targets), logits.is_cuda)
    if pc is not None and mode == ParallelMode.TENSOR_3D and pc.tensor_parallel_size > 1:
        # the 3-D head gathers full logits on every rank; the plain loss then runs replicated
        flat = logits[..., :orig_vocab].reshape(-1, orig_vocab).float()
        return LossResult(F.cross_entropy(flat, targets.reshape(-1), ignore_index=ignore_index), False)
    # unsharded vocabulary: same kernel path with a group of one
    fn = onn.VocabParallelCrossEntropyLoss1D(parallel_context=None, ignore_index=ignore_index)
    fn.orig_vocab_size = orig_vocab
    return LossResult(fn(logits, targets), logits.is_cuda)


def chunked_head_loss(model, hidden, head, labels, chunk_size: int, ignore_index: int = -100):
    """Next-token loss straight from the final hidden states: LM head and cross-entropy run chunk by chunk
    (:func:`oslo_b200.ops.linear_cross_entropy.linear_cross_entropy`), the ``[tokens, vocab]`` logits never exist.  Returns
    ``None`` when the head is not a plain (unsharded, bias-free) linear, in which case the caller takes the usual path."""
    if type(head) not in (torch.nn.Linear, onn.Linear) or getattr(head, "bias", None) is not None:
        return None
    pc = getattr(model, "parallel_context", None)
    if pc is not None and pc.tensor_parallel_size > 1:
        return None
    from oslo_b200.ops.linear_cross_entropy import linear_cross_entropy

    return linear_cross_entropy(hidden, head.weight, shift_labels(labels, ignore_index), chunk_size, ignore_index,
                                orig_vocab_size=model.config.vocab_size)
