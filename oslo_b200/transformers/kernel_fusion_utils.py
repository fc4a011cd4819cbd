"""Model surgery helpers that switch Hugging Face models to the fused kernels.

``fused_no_repeat_ngram_logits_processor(model)``: generation uses the n-gram blocking kernel;
``fused_rms_norm(model)``: every T5 / Llama style RMS norm module becomes ``FusedRMSNorm``;
``fused_layer_norm(model)``: every ``nn.LayerNorm`` becomes ``FusedLayerNorm``.
Parity: oslo/transformers/kernel_fusion_utils.py:7-87.
"""
from __future__ import annotations

import torch.nn as nn

import oslo_b200.nn as onn
from oslo_b200.nn.ngram_repeat_block import fused_no_repeat_ngram_logits_processor  # noqa: F401

_RMS_CLASS_NAMES = ("T5LayerNorm", "LlamaRMSNorm", "MT5LayerNorm", "MistralRMSNorm")


def _swap(model: nn.Module, predicate, factory) -> int:
    n = 0
    for parent in model.modules():
        for name, child in list(parent.named_children()):
            if predicate(child):
                setattr(parent, name, factory(child))
                n += 1
    return n


def fused_rms_norm(model: nn.Module) -> nn.Module:
    def make(old):
        eps = getattr(old, "variance_epsilon", getattr(old, "eps", 1e-6))
        new = onn.FusedRMSNorm(old.weight.shape[0], eps=eps, dtype=old.weight.dtype, device=old.weight.device)
        new.weight = old.weight
        return new

    _swap(model, lambda m: m.__class__.__name__ in _RMS_CLASS_NAMES, make)
    return model


def fused_layer_norm(model: nn.Module) -> nn.Module:
    def make(old):
        new = onn.FusedLayerNorm(old.normalized_shape, eps=old.eps, elementwise_affine=old.elementwise_affine)
        if old.elementwise_affine:
            new.weight, new.bias = old.weight, old.bias
        return new

    _swap(model, lambda m: type(m) is nn.LayerNorm, make)
    return model
