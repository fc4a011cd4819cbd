"""Functional entry points of the fused ops (CUDA kernels on GPU, torch on CPU).

Parity: oslo/torch/nn/modules/functional.py:23-298.
"""
from oslo_b200.ops.activation import (  # noqa: F401
    bias_act,
    bias_dropout_add,
    bias_gelu,
    fused_bias_dropout,
    fused_bias_gelu,
    fused_gelu,
    swiglu,
)
from oslo_b200.ops.attention import attention, qkv_attention  # noqa: F401
from oslo_b200.ops.norm import layer_norm as fused_layer_norm  # noqa: F401
from oslo_b200.ops.norm import rms_norm as fused_rms_norm  # noqa: F401
from oslo_b200.ops.softmax import apply_rope, rope_tables, scale_mask_softmax  # noqa: F401


def fused_layer_norm_affine(input, weight, bias, normalized_shape, eps=1e-6):
    return fused_layer_norm(input, normalized_shape, weight, bias, eps)


def fused_rms_norm_affine(input, weight, normalized_shape, eps=1e-6):
    return fused_rms_norm(input, normalized_shape, weight, eps)


# mixed-dtype variants: parameters kept in fp32 while activations are fp16 / bf16
mixed_dtype_fused_layer_norm_affine = fused_layer_norm_affine
mixed_dtype_fused_rms_norm_affine = fused_rms_norm_affine
