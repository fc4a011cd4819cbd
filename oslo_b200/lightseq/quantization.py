"""Fake-quantisation modules for int8 quantisation-aware training (kept as the short import path).

The toolkit itself lives in :mod:`oslo_b200.lightseq.pytorch_quantization`; this module re-exports the two classes the
LightSeq-style layers use and the real int8 quantisation used by the exporter (kernels: ``csrc/lightseq_sm100a.cu``).
"""
from __future__ import annotations

import torch

from .pytorch_quantization import QuantLinear, TensorQuantizer  # noqa: F401


def quantize_int8(x: torch.Tensor, amax: torch.Tensor):
    """Real int8 quantisation (for export): returns ``(int8 tensor, scale)``."""
    scale = amax.clamp_min(1e-12) / 127.0
    return torch.clamp(torch.round(x / scale), -127, 127).to(torch.int8), scale
