"""``FusedBiasDropout``: ``dropout(x + bias)`` (+ residual) in one kernel.

Parity: oslo/torch/nn/modules/dropout.py:9-11.
"""
import torch.nn as nn

from oslo_b200.ops.activation import bias_dropout_add


class FusedBiasDropout(nn.Dropout):
    def forward(self, input, bias=None, residual=None):
        return bias_dropout_add(input, bias, residual, self.p, self.training)
