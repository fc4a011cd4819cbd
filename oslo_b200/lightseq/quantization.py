"""Fake-quantisation modules for int8 quantisation-aware training.

``TensorQuantizer`` (symmetric per-tensor or per-channel, max or moving-average calibration, straight-through
gradient with clipping mask) and ``QuantLinear`` follow the subset of NVIDIA's pytorch_quantization toolkit that
LightSeq's quantised layers use (oslo/lightseq2/training/pytorch_quantization/*, kernels in
csrc/kernels/cuda/quantize_kernels.cu).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F


class _FakeQuant(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, amax, bits):
        qmax = 2.0 ** (bits - 1) - 1
        scale = amax.clamp_min(1e-12) / qmax
        ctx.save_for_backward((x.abs() <= amax))
        return torch.clamp(torch.round(x / scale), -qmax, qmax) * scale

    @staticmethod
    def backward(ctx, g):
        (inside,) = ctx.saved_tensors
        return g * inside, None, None


class TensorQuantizer(nn.Module):
    def __init__(self, num_bits: int = 8, axis: Optional[int] = None, momentum: float = 0.99, learn_amax: bool = False):
        super().__init__()
        self.num_bits, self.axis, self.momentum = num_bits, axis, momentum
        self.calibrating, self.enabled = True, True
        self.register_buffer("amax", torch.tensor(0.0))
        self.learn_amax = learn_amax

    def _observe(self, x):
        if self.axis is None:
            cur = x.detach().abs().max()
        else:
            dims = [d for d in range(x.dim()) if d != self.axis % x.dim()]
            cur = x.detach().abs().amax(dim=dims, keepdim=True)
        if self.amax.numel() == 1 and float(self.amax.max()) == 0.0:
            self.amax = cur.clone()
        else:
            self.amax = self.momentum * self.amax + (1 - self.momentum) * cur

    def forward(self, x):
        if not self.enabled:
            return x
        if self.calibrating and self.training:
            self._observe(x)
        return _FakeQuant.apply(x, self.amax.to(x.dtype), self.num_bits)


class QuantLinear(nn.Linear):
    """Linear layer with fake-quantised input and (per-output-channel) weight."""

    def __init__(self, in_features, out_features, bias=True, num_bits: int = 8):
        super().__init__(in_features, out_features, bias)
        self.input_quantizer = TensorQuantizer(num_bits)
        self.weight_quantizer = TensorQuantizer(num_bits, axis=0)

    def forward(self, x):
        return F.linear(self.input_quantizer(x), self.weight_quantizer(self.weight), self.bias)


def quantize_int8(x: torch.Tensor, amax: torch.Tensor):
    """Real int8 quantisation (for export): returns ``(int8 tensor, scale)``."""
    scale = amax.clamp_min(1e-12) / 127.0
    return torch.clamp(torch.round(x / scale), -127, 127).to(torch.int8), scale
