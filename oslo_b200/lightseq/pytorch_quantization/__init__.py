"""Quantisation-aware-training toolkit: descriptors, calibrators, quantiser module, quantised layers, module swapping and
optimizer helpers (parity: oslo/lightseq2/training/pytorch_quantization/*).

Typical use::

    from oslo_b200.lightseq import pytorch_quantization as pq
    pq.replace_with_quant(model, skip=["lm_head"])      # or pq.quant_modules.initialize() before building the model
    pq.collect_stats(model, calibration_batches, 8)     # calibrators see activations, quantisation off
    pq.compute_amax(model, "percentile", percentile=99.99)
    pq.qat_mode(model)                                  # fine-tune with fake quantisation
"""
from . import calib, nn, optim, quant_modules, tensor_quant  # noqa: F401
from .calib import HistogramCalibrator, MaxCalibrator, calibrate_weights
from .nn import (Clip, QuantConv1d, QuantConv2d, QuantConv3d, QuantEmbedding, QuantLinear, QuantMatmul, QuantSelfAttention,
                 TensorQuantizer, collect_stats, compute_amax, disable_quant, enable_quant, ptq_mode, qat_mode)
from .optim import freeze_parameters, group_parameters, match_parameters, quant_weight_inplace
from .quant_modules import deactivate, initialize, quantized_construction, replace_with_quant
from .tensor_quant import (QuantDescriptor, ScaledQuantDescriptor, fake_affine_tensor_quant, fake_tensor_quant, reduce_amax,
                           tensor_quant as tensor_quant_fn)

__all__ = ["calib", "nn", "optim", "quant_modules", "tensor_quant", "QuantDescriptor", "ScaledQuantDescriptor", "TensorQuantizer",
           "QuantLinear", "QuantConv1d", "QuantConv2d", "QuantConv3d", "QuantEmbedding", "QuantMatmul", "QuantSelfAttention", "Clip",
           "MaxCalibrator", "HistogramCalibrator", "calibrate_weights", "collect_stats", "compute_amax", "enable_quant",
           "disable_quant", "qat_mode", "ptq_mode", "initialize", "deactivate", "quantized_construction", "replace_with_quant",
           "match_parameters", "group_parameters", "freeze_parameters", "quant_weight_inplace", "fake_tensor_quant",
           "fake_affine_tensor_quant", "tensor_quant_fn", "reduce_amax"]
