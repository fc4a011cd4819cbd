"""Loss helpers shared by the task heads of the encoder and encoder-decoder models."""
from __future__ import annotations

import torch
import torch.nn.functional as F


def classification_loss(logits, labels, num_labels: int):
    """Regression (one label, MSE), single-label (cross-entropy) or multi-label (BCE) loss, chosen like the Hugging Face
    heads do from ``num_labels`` and the label dtype; ``None`` without labels."""
    if labels is None:
        return None
    if num_labels == 1:
        return F.mse_loss(logits.squeeze(-1).float(), labels.squeeze(-1).float() if labels.dim() > 1 else labels.float())
    if labels.dtype in (torch.long, torch.int):
        return F.cross_entropy(logits.view(-1, num_labels).float(), labels.view(-1))
    return F.binary_cross_entropy_with_logits(logits.float(), labels.float())


def qa_loss(start_logits, end_logits, start_positions, end_positions):
    """Mean of the start and end cross-entropies; positions outside the sequence are ignored."""
    if start_positions is None or end_positions is None:
        return None
    s = start_logits.shape[1]
    sp, ep = start_positions.view(-1).clamp(0, s), end_positions.view(-1).clamp(0, s)
    return 0.5 * (F.cross_entropy(start_logits.float(), sp, ignore_index=s) + F.cross_entropy(end_logits.float(), ep, ignore_index=s))
