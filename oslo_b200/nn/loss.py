"""Cross-entropy losses for vocabulary-sharded logits in every tensor-parallel mode.

``VocabParallelCrossEntropyLoss1D`` takes logits ``[..., V/tp]`` and global targets; the 2D / 2.5D
variants take logits whose vocabulary is sharded over the ROW group and whose batch is sharded over
COL, with targets for the full batch; ``CrossEntropyLoss{2D,2p5D,3D}`` are plain cross-entropy on
batch-sharded inputs followed by the cross-rank mean.  All return the mean over non-ignored tokens.

Parity: oslo/torch/nn/modules/loss.py:14-570.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from oslo_b200.distributed import ParallelMode, comm
from oslo_b200.ops.loss import vocab_parallel_cross_entropy


class _AllReduceSum(torch.autograd.Function):
    """Sum over a group in forward; gradient passes through unchanged (each rank owns its term)."""

    @staticmethod
    def forward(ctx, x, pc, mode):
        return comm.all_reduce(x.clone(), parallel_context=pc, parallel_mode=mode)

    @staticmethod
    def backward(ctx, g):
        return g, None, None


def _mean_over_valid(loss, targets, ignore_index, pc=None, batch_modes=()):
    """Mean of per-token losses over non-ignored tokens; the tokens are spread over the ``batch_modes`` groups."""
    valid = (targets != ignore_index)
    total = loss.sum()
    count = valid.sum().to(loss.dtype)
    for mode in batch_modes:
        if pc is not None and pc.get_world_size(mode) > 1:
            total = _AllReduceSum.apply(total, pc, mode)
            count = comm.all_reduce(count.clone(), parallel_context=pc, parallel_mode=mode)
    return total / count.clamp(min=1)


class VocabParallelCrossEntropyLoss1D(nn.Module):
    def __init__(self, reduce_mean=True, ignore_index=-100, parallel_context=None):
        super().__init__()
        self.reduce_mean = reduce_mean
        self.ignore_index = ignore_index
        self.parallel_context = parallel_context

    def forward(self, logits, targets):
        valid_vocab = getattr(self, "orig_vocab_size", None)
        loss = vocab_parallel_cross_entropy(logits, targets, self.parallel_context, ParallelMode.TENSOR_1D,
                                            self.ignore_index, valid_vocab)
        if not self.reduce_mean:
            return loss
        return _mean_over_valid(loss, targets, self.ignore_index)


class _VocabParallelCrossEntropyLossND(nn.Module):
    vocab_mode: ParallelMode
    batch_modes = ()

    def __init__(self, reduce_mean=True, ignore_index=-100, parallel_context=None):
        super().__init__()
        self.reduce_mean = reduce_mean
        self.ignore_index = ignore_index
        self.parallel_context = parallel_context

    def forward(self, logits, targets):
        pc = self.parallel_context
        for mode in self.batch_modes:
            targets = comm.scatter(targets, dim=0, parallel_context=pc, parallel_mode=mode)
        valid_vocab = getattr(self, "orig_vocab_size", None)
        loss = vocab_parallel_cross_entropy(logits, targets, pc, self.vocab_mode, self.ignore_index, valid_vocab)
        if not self.reduce_mean:
            return loss
        return _mean_over_valid(loss, targets, self.ignore_index, pc, self.batch_modes)


class VocabParallelCrossEntropyLoss2D(_VocabParallelCrossEntropyLossND):
    vocab_mode = ParallelMode.TENSOR_2D_ROW
    batch_modes = (ParallelMode.TENSOR_2D_COL,)


class VocabParallelCrossEntropyLoss2p5D(_VocabParallelCrossEntropyLossND):
    vocab_mode = ParallelMode.TENSOR_2P5D_ROW
    batch_modes = (ParallelMode.TENSOR_2P5D_DEP, ParallelMode.TENSOR_2P5D_COL)


class _CrossEntropyLossND(nn.Module):
    batch_modes = ()

    def __init__(self, reduce_mean=True, ignore_index=-100, parallel_context=None, *args, **kwargs):
        super().__init__()
        self.reduce_mean = reduce_mean
        self.ignore_index = ignore_index
        self.parallel_context = parallel_context

    def forward(self, logits, targets):
        pc = self.parallel_context
        for mode in self.batch_modes:
            targets = comm.scatter(targets, dim=0, parallel_context=pc, parallel_mode=mode)
        loss = F.cross_entropy(logits.reshape(-1, logits.shape[-1]).float(), targets.reshape(-1),
                               ignore_index=self.ignore_index, reduction="none")
        if not self.reduce_mean:
            return loss
        flat_t = targets.reshape(-1)
        total, count = loss.sum(), (flat_t != self.ignore_index).sum().to(loss.dtype)
        for mode in self.batch_modes:
            if pc.get_world_size(mode) > 1:
                total = _AllReduceSum.apply(total, pc, mode)
                count = comm.all_reduce(count.clone(), parallel_context=pc, parallel_mode=mode)
        return total / count.clamp(min=1)


class CrossEntropyLoss2D(_CrossEntropyLossND):
    batch_modes = (ParallelMode.TENSOR_2D_COL,)


class CrossEntropyLoss2p5D(_CrossEntropyLossND):
    batch_modes = (ParallelMode.TENSOR_2P5D_DEP, ParallelMode.TENSOR_2P5D_COL)


class CrossEntropyLoss3D(_CrossEntropyLossND):
    batch_modes = (ParallelMode.TENSOR_3D_WEIGHT, ParallelMode.TENSOR_3D_INPUT)
