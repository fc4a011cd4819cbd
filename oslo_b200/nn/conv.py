"""GPT-2 style ``Conv1D`` (a linear layer whose weight is stored ``[in, out]``).

Parity: ``oslo/torch/nn/modules/conv.py:5-42``.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from oslo_b200.ops.gemm import linear as _linear


class Conv1D(nn.Module):
    def __init__(self, nf: int, nx: int, skip_bias_add: bool = False, dtype=None, device=None):
        super().__init__()
        self.nf = nf
        self.skip_bias_add = skip_bias_add
        w = torch.empty(nx, nf, dtype=dtype, device=device)
        nn.init.normal_(w, std=0.02)
        self.weight = nn.Parameter(w)
        self.bias = nn.Parameter(torch.zeros(nf, dtype=dtype, device=device))

    def forward(self, x):
        # weight.t() is an MN-major operand for the GEMM kernel: no transposition copy
        if self.skip_bias_add:
            return _linear(x, self.weight.t()), self.bias
        return _linear(x, self.weight.t(), self.bias)
