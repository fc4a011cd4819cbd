"""``NGramRepeatBlock``: forbid repeating any n-gram during beam search (CUDA kernel or a vectorised torch fallback),
and a Hugging Face ``LogitsProcessor`` built on it.

Parity: oslo/torch/nn/modules/ngram_repeat_block.py:41-122, oslo/transformers/kernel_fusion_utils.py:7-68.
"""
from __future__ import annotations

import ctypes

import torch
import torch.nn as nn

from oslo_b200.ops import _lib

_DT = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


def ngram_repeat_block_reference(tokens, lprobs, step, no_repeat_ngram_size):
    n = no_repeat_ngram_size
    rows = tokens.shape[0]
    if step + 1 < n:
        return lprobs
    ctx = tokens[:, step - n + 2 : step + 1] if n > 1 else tokens[:, :0]
    for r in range(rows):
        seq = tokens[r, : step + 1].tolist()
        tail = ctx[r].tolist()
        for s in range(0, step + 2 - n):
            if seq[s : s + n - 1] == tail:
                lprobs[r, seq[s + n - 1]] = float("-inf")
    return lprobs


class NGramRepeatBlock(nn.Module):
    def forward(self, tokens, lprobs, bsz, step, beam_size, no_repeat_ngram_size):
        """``tokens [bsz*beam, max_len]`` (int64), ``lprobs [bsz*beam, vocab]``; ``step`` = index of the last token."""
        assert tokens.shape[0] == bsz * beam_size == lprobs.shape[0]
        if lprobs.is_cuda and _lib.has_cuda_kernels() and lprobs.dtype in _DT and lprobs.is_contiguous():
            tok = tokens.to(torch.int64).contiguous()
            rc = _lib.cuda_lib().oslo_ngram_repeat_block(
                _lib.ptr(tok), _lib.ptr(lprobs), ctypes.c_int(tok.shape[0]), ctypes.c_int(tok.shape[1]), ctypes.c_int(step),
                ctypes.c_int(lprobs.shape[1]), ctypes.c_int(no_repeat_ngram_size), ctypes.c_int(_DT[lprobs.dtype]),
                _lib.stream_ptr())
            if rc:
                raise RuntimeError(f"oslo_ngram_repeat_block failed ({rc})")
            return lprobs
        return ngram_repeat_block_reference(tokens, lprobs, step, no_repeat_ngram_size)


class FusedNoRepeatNGramLogitsProcessor:
    """Drop-in for ``transformers.NoRepeatNGramLogitsProcessor`` (callable ``(input_ids, scores) -> scores``)."""

    def __init__(self, ngram_size: int, batch_size: int = None, beam_size: int = None):
        if ngram_size <= 0:
            raise ValueError("ngram_size must be positive")
        self.ngram_size, self.batch_size, self.beam_size = ngram_size, batch_size, beam_size
        self.block = NGramRepeatBlock()

    def __call__(self, input_ids, scores):
        rows = input_ids.shape[0]
        beam = self.beam_size or 1
        return self.block(input_ids, scores, rows // beam, input_ids.shape[1] - 1, beam, self.ngram_size)


def fused_no_repeat_ngram_logits_processor(model):
    """Make ``model.generate`` use the fused n-gram blocker when ``no_repeat_ngram_size`` is set."""
    orig = getattr(model, "_get_logits_processor", None)
    if orig is None:
        return model

    def patched(*args, **kwargs):
        processors = orig(*args, **kwargs)
        for i, p in enumerate(processors):
            if p.__class__.__name__ == "NoRepeatNGramLogitsProcessor":
                processors[i] = FusedNoRepeatNGramLogitsProcessor(p.ngram_size)
        return processors

    model._get_logits_processor = patched
    return model
