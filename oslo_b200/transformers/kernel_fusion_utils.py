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


def fused_linear(model: nn.Module) -> nn.Module:
    """Every plain ``nn.Linear`` computes through the tcgen05 GEMM (forward, dX and dW) instead of cuBLAS."""
    import torch

    def make(old):
        new = onn.Linear.__new__(onn.Linear)
        nn.Module.__init__(new)
        new.in_features, new.out_features, new.skip_bias_add = old.in_features, old.out_features, False
        new.weight, new.bias = old.weight, old.bias
        return new

    _swap(model, lambda m: type(m) is torch.nn.Linear, make)
    return model


_ATTENTION_NAME = "oslo_b200"


def _oslo_attention_forward(module, query, key, value, attention_mask, dropout: float = 0.0, scaling=None, is_causal=None,
                            **kwargs):
    """Hugging Face attention-interface function backed by the fused tcgen05 attention kernels.

    ``query / key / value`` arrive as ``[batch, heads, seq, head_dim]``; the result is ``[batch, seq, heads, head_dim]`` as
    the interface expects.  Calls the kernels cannot take (an explicit mask, attention dropout in training, a key length
    different from the query length) go to the stock scaled-dot-product implementation."""
    from transformers.integrations.sdpa_attention import sdpa_attention_forward

    from oslo_b200.ops.attention import attention

    b, h, s, d = query.shape
    if attention_mask is not None or (dropout and module.training) or key.shape[2] != s:
        return sdpa_attention_forward(module, query, key, value, attention_mask, dropout=dropout, scaling=scaling,
                                      is_causal=is_causal, **kwargs)
    if key.shape[1] != h:  # grouped-query attention: repeat the key / value heads
        rep = h // key.shape[1]
        key, value = key.repeat_interleave(rep, dim=1), value.repeat_interleave(rep, dim=1)
    causal = is_causal if is_causal is not None else (s > 1 and getattr(module, "is_causal", True))
    out = attention(query.transpose(1, 2), key.transpose(1, 2), value.transpose(1, 2), causal=bool(causal), scale=scaling)
    return out.view(b, s, h, d), None


def fused_attention(model: nn.Module) -> nn.Module:
    """Route the attention of a Hugging Face model through the fused attention kernels: registers the
    ``"oslo_b200"`` implementation with the transformers attention interface and selects it in the model's config (the
    reference's forks hard-wire their fused softmax / LightSeq attention per model family,
    oslo/transformers/models/bert/modeling_bert.py:349-401)."""
    from transformers import AttentionInterface

    AttentionInterface.register(_ATTENTION_NAME, _oslo_attention_forward)
    cfg = getattr(model, "config", None)
    if cfg is not None:
        cfg._attn_implementation = _ATTENTION_NAME
        for sub in model.modules():
            if getattr(sub, "config", None) is not None and sub.config is not cfg and hasattr(sub.config, "_attn_implementation"):
                sub.config._attn_implementation = _ATTENTION_NAME
    return model


def fuse_all(model: nn.Module) -> nn.Module:
    """LayerNorm / RMSNorm, linears and attention of a stock Hugging Face model on this library's kernels."""
    return fused_attention(fused_linear(fused_layer_norm(fused_rms_norm(model))))
