"""Linear-chain conditional random field layer: negative log-likelihood for training, Viterbi decoding for inference.

Counterpart of the CRF layer and kernels of the reference's LightSeq subset (oslo/lightseq2/csrc/layers_new/crf_layer.cpp,
csrc/kernels/cuda/crf.cu; oracle csrc/tests/cuda/torch_crf.py).  The recursions over the sequence are written as batched
tensor operations over ``[batch, tags, tags]`` (one log-sum-exp / max per time step), so they run on the GPU through
PyTorch; there is no per-token Python loop over the batch or the tags.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.nn as nn


class LSCRFLayer(nn.Module):
    """``forward(emissions, tags, mask)`` -> summed (or mean) negative log-likelihood; ``decode(emissions, mask)`` ->
    best tag sequences.  ``emissions``: ``[batch, seq, num_tags]`` (batch first), ``mask``: ``[batch, seq]`` with the first
    position of every sequence on."""

    def __init__(self, num_tags: int):
        super().__init__()
        if num_tags <= 0:
            raise ValueError("num_tags must be positive")
        self.num_tags = num_tags
        self.start_transitions = nn.Parameter(torch.empty(num_tags))
        self.end_transitions = nn.Parameter(torch.empty(num_tags))
        self.transitions = nn.Parameter(torch.empty(num_tags, num_tags))  # [from, to]
        for p in self.parameters():
            nn.init.uniform_(p, -0.1, 0.1)

    def forward(self, emissions, tags, mask: Optional[torch.Tensor] = None, reduction: str = "sum"):
        if mask is None:
            mask = torch.ones_like(tags, dtype=torch.bool)
        mask = mask.bool()
        if not bool(mask[:, 0].all()):
            raise ValueError("the first position of every sequence must be unmasked")
        e = emissions.float()
        nll = self._normalizer(e, mask) - self._score(e, tags, mask)
        if reduction == "none":
            return nll
        if reduction == "sum":
            return nll.sum()
        if reduction == "mean":
            return nll.mean()
        if reduction == "token_mean":
            return nll.sum() / mask.sum()
        raise ValueError(f"unknown reduction {reduction}")

    def _score(self, e, tags, mask):
        b, s, _ = e.shape
        m = mask.float()
        first = self.start_transitions[tags[:, 0]] + e[:, 0].gather(1, tags[:, :1]).squeeze(1)
        trans = self.transitions[tags[:, :-1], tags[:, 1:]]                      # [b, s-1]
        emit = e[:, 1:].gather(2, tags[:, 1:].unsqueeze(-1)).squeeze(-1)         # [b, s-1]
        body = ((trans + emit) * m[:, 1:]).sum(1)
        last = tags.gather(1, (mask.long().sum(1) - 1).unsqueeze(1)).squeeze(1)
        return first + body + self.end_transitions[last]

    def _normalizer(self, e, mask):
        alpha = self.start_transitions + e[:, 0]                                   # [b, tags]
        for t in range(1, e.shape[1]):
            nxt = torch.logsumexp(alpha.unsqueeze(2) + self.transitions.unsqueeze(0), dim=1) + e[:, t]
            alpha = torch.where(mask[:, t].unsqueeze(1), nxt, alpha)
        return torch.logsumexp(alpha + self.end_transitions, dim=1)

    @torch.no_grad()
    def decode(self, emissions, mask: Optional[torch.Tensor] = None) -> List[List[int]]:
        e = emissions.float()
        b, s, _ = e.shape
        if mask is None:
            mask = torch.ones(b, s, dtype=torch.bool, device=e.device)
        mask = mask.bool()
        score = self.start_transitions + e[:, 0]
        back = []
        for t in range(1, s):
            cand = score.unsqueeze(2) + self.transitions.unsqueeze(0)             # [b, from, to]
            best, idx = cand.max(dim=1)
            nxt = best + e[:, t]
            keep = mask[:, t].unsqueeze(1)
            score = torch.where(keep, nxt, score)
            # masked steps point back at themselves so the walk below passes straight through them
            back.append(torch.where(keep, idx, torch.arange(self.num_tags, device=e.device).expand(b, -1)))
        score = score + self.end_transitions
        last = score.argmax(dim=1)
        path = [last]
        for idx in reversed(back):
            last = idx.gather(1, last.unsqueeze(1)).squeeze(1)
            path.append(last)
        full = torch.stack(path[::-1], dim=1)                                      # [b, s]
        lengths = mask.long().sum(1).tolist()
        return [full[i, : lengths[i]].tolist() for i in range(b)]


__all__ = ["LSCRFLayer"]
