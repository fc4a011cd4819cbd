"""Layer-id interface: create a layer under an integer id, bind its parameters and gradients to slices of flat buffers,
then run forward / backward by id.

This is the calling convention of the reference's LightSeq extension modules (oslo/lightseq2/csrc/pybind/pybind_layer.cpp:
``create_transformer_encoder_layer(layer_id, ...)``, ``transformer_encoder_layer_fw / _bw(layer_id, ...)``,
``assign_layer_weight_grad(weights, grads, "TransformerEncoderLayer", layer_id)``), which frameworks such as fairseq drive
with one flat parameter tensor per layer.  Here the registry holds ordinary modules of :mod:`oslo_b200.lightseq.layers`;
``assign_layer_weight_grad`` re-points every parameter (and its ``.grad``) at a slice of the caller's flat buffers, so an
optimizer that updates the flat tensor updates the layer, and the layer's backward accumulates into the flat gradient.
"""
from __future__ import annotations

from typing import Dict, List, Tuple

import torch

from .layers import (LSCrossEntropyLayer, LSLayerConfig, LSTransformerDecoderLayer, LSTransformerEmbeddingLayer,
                     LSTransformerEncoderLayer)

_KINDS = {"TransformerEncoderLayer": LSTransformerEncoderLayer, "TransformerDecoderLayer": LSTransformerDecoderLayer,
          "TransformerEmbeddingLayer": LSTransformerEmbeddingLayer, "CrossEntropyLayer": LSCrossEntropyLayer}
_layers: Dict[Tuple[str, int], torch.nn.Module] = {}
_saved: Dict[Tuple[str, int], tuple] = {}


def _create(kind: str, layer_id: int, dtype=torch.float32, device=None, **cfg):
    extra = {}
    if kind == "TransformerEncoderLayer":
        extra["causal"] = bool(cfg.pop("mask_future_tokens", False))
    cfg["pre_layer_norm"] = cfg.pop("is_pre_ln", cfg.get("pre_layer_norm", True))
    if "hidden_dim" in cfg:
        cfg["hidden_size"] = cfg.pop("hidden_dim")
    if "num_heads" in cfg:
        cfg["nhead"] = cfg.pop("num_heads")
    layer = _KINDS[kind](LSLayerConfig(**cfg), **extra)
    layer = layer.to(device=device, dtype=dtype) if device is not None else layer.to(dtype=dtype)
    _layers[(kind, layer_id)] = layer
    return 0


def create_transformer_encoder_layer(layer_id: int, **cfg) -> int:
    return _create("TransformerEncoderLayer", layer_id, **cfg)


def create_transformer_decoder_layer(layer_id: int, **cfg) -> int:
    return _create("TransformerDecoderLayer", layer_id, **cfg)


def create_transformer_embedding_layer(layer_id: int, **cfg) -> int:
    return _create("TransformerEmbeddingLayer", layer_id, **cfg)


def create_cross_entropy_layer(layer_id: int, **cfg) -> int:
    return _create("CrossEntropyLayer", layer_id, **cfg)


def get_layer(kind: str, layer_id: int) -> torch.nn.Module:
    return _layers[(kind, layer_id)]


def layer_param_numel(kind: str, layer_id: int) -> int:
    """Elements of the flat buffer that :func:`assign_layer_weight_grad` expects."""
    return sum(p.numel() for p in _layers[(kind, layer_id)].parameters())


def assign_layer_weight_grad(weights: torch.Tensor, grads: torch.Tensor, kind: str, layer_id: int) -> int:
    """Bind the layer's parameters to consecutive slices of ``weights`` (their current values are copied in first) and their
    gradients to the same slices of ``grads``."""
    layer = _layers[(kind, layer_id)]
    need = sum(p.numel() for p in layer.parameters())
    if weights.numel() != need or grads.numel() != need:
        raise ValueError(f"flat buffers must hold {need} elements, got {weights.numel()} / {grads.numel()}")
    off = 0
    with torch.no_grad():
        for p in layer.parameters():
            n = p.numel()
            w = weights.view(-1)[off : off + n].view_as(p)
            w.copy_(p)
            p.data = w
            p.grad = grads.view(-1)[off : off + n].view_as(p)
            off += n
    return 0


def _fw(kind, layer_id, inputs: List[torch.Tensor], training_mode: bool, call):
    layer = _layers[(kind, layer_id)]
    layer.train(training_mode)
    leaves = [t.detach().requires_grad_(t.is_floating_point() and training_mode) for t in inputs]
    with torch.set_grad_enabled(training_mode):
        out = call(layer, *leaves)
    _saved[(kind, layer_id)] = (leaves, out)
    return [out.detach()] if torch.is_tensor(out) else [o.detach() for o in out]


def _bw(kind, layer_id, grad_outputs: List[torch.Tensor]):
    leaves, out = _saved.pop((kind, layer_id))
    outs = [out] if torch.is_tensor(out) else list(out)
    torch.autograd.backward(outs, grad_outputs)  # parameter gradients accumulate into the bound flat slices
    return [t.grad for t in leaves if t.requires_grad]


def transformer_encoder_layer_fw(layer_id, input, input_mask=None, training_mode=True, *unused):
    mask = None if input_mask is None or not bool(input_mask.any()) else input_mask.bool()
    return _fw("TransformerEncoderLayer", layer_id, [input], training_mode, lambda l, x: l(x, mask))


def transformer_encoder_layer_bw(layer_id, grad_output, *unused):
    return _bw("TransformerEncoderLayer", layer_id, [grad_output])


def transformer_decoder_layer_fw(layer_id, dec_input, enc_output, enc_mask=None, training_mode=True, *unused):
    mask = None if enc_mask is None or not bool(enc_mask.any()) else enc_mask.bool()
    return _fw("TransformerDecoderLayer", layer_id, [dec_input, enc_output], training_mode, lambda l, d, e: l(d, e, mask))


def transformer_decoder_layer_bw(layer_id, grad_output, *unused):
    return _bw("TransformerDecoderLayer", layer_id, [grad_output])


def transformer_embedding_layer_fw(layer_id, input_ids, step=0, training_mode=True):
    return _fw("TransformerEmbeddingLayer", layer_id, [input_ids], training_mode, lambda l, ids: l(ids, step=step))


def transformer_embedding_layer_bw(layer_id, grad_output, *unused):
    return _bw("TransformerEmbeddingLayer", layer_id, [grad_output])


def cross_entropy_layer_fw(layer_id, logits, targets):
    return _fw("CrossEntropyLayer", layer_id, [logits, targets], True, lambda l, x, t: l(x, t))


def cross_entropy_layer_bw(layer_id, grad_loss):
    leaves, out = _saved.pop(("CrossEntropyLayer", layer_id))
    out[0].backward(grad_loss)
    return [leaves[0].grad]


def clear() -> None:
    _layers.clear()
    _saved.clear()


__all__ = [n for n in globals() if n.startswith(("create_", "transformer_", "cross_entropy_", "assign_", "get_layer", "layer_param", "clear"))]
